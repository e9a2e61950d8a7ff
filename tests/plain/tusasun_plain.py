"""Plain, slow Tusasun: whole sequences, no cache, one function per mechanism.

The oracle of the Tusasun tests.  It shares no code with toyinfer_b200: the configuration is a
dict as config.json holds it, the weights a dict of tensors by checkpoint name, and every
mechanism is written token by token with elementary torch operations in float64.

The design in this file's notation (one row per token; W applies as W x; weights [out, in]):

* streams:   X [n, width], n = ``streams`` copies of the embedding row at the start.  A sublayer f
             with constants a [n] (read), M [n, n] (carry, [from, to]), b [n] (write) and a
             per-channel scale s does:  u = sum_i a_i X_i;  y = s * f(norm(u));
             X_j <- sum_i M_ij X_i + b_j y  for all j from the old X.  Every layer has two such
             sublayers (mixer, then feed-forward).  At the end x = sum_i X_i.
* norm:      v / sqrt(mean(v^2) + eps) * (1 + w)
* loop:      layers [start, stop) run ``times`` times with the same weights, then the rest
* rglru:     two branches of ``width`` channels: p = gelu_tanh(Wy h + by); c = Wx h + bx, then a
             causal convolution per channel over the last ``conv`` rows (with bias); the
             channels are cut into ``blocks`` parts, each with two square gate matrices:
             r = sigmoid(Ra c + ra), i = sigmoid(Ri c + ri); a = exp(-8 r softplus(lam));
             S <- a S + sqrt(1 - a^2) (i c);  out = Wo (S p)
* attention: q, k, v with biases; q and k normed per head (plain weight); score =
             cap tanh(q.k scale / cap) + table[bucket(i - j), head]; causal softmax; Wo with bias.
             bucket(d) = d below half = rows/2, else min(rows - 1, half + floor(ln(d / half) /
             ln(far / half) (rows - half)))
* channel_delta: q, k (kv_heads x dim) and v (heads x vdim) each through a causal convolution
             per channel (no bias) and silu; q, k made unit vectors per head (q also times
             dim^-1/2); beta = sigmoid(Wb h) per head; decay per head and key channel
             g = exp(-exp(A_h) softplus(Wa2 Wa1 h + dt));  per head, with S [dim, vdim]:
             S <- g S (rows); e = beta (v - S^T k); S <- S + k e^T; o = S^T q; then o / rms(o)
             times a weight [vdim] times sigmoid(Wg2 Wg1 h), and Wo
* experts:   z = Wr h; the ``top`` largest sigmoid(z) choose experts; each runs
             Wdown relu(Wup (sigmoid(z_e) h))^2; a shared expert of the same form runs for every
             token, times sigmoid(wsg . h)
* output:    logits = head (norm_final(x))
"""
from __future__ import annotations

import math
from typing import Dict, List, Sequence

import torch

F64 = torch.float64


def one_plus_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.to(F64)
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * (1.0 + w.to(F64))


def plain_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.to(F64)
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w.to(F64)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * sigmoid(z)


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias=None) -> torch.Tensor:
    """x [T, C]; taps [C, n], the last column weighs the current row; zeros before row 0."""
    T, C = x.shape
    n = taps.shape[1]
    out = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        for j in range(n):
            s = t - (n - 1 - j)
            if s >= 0:
                out[t] += taps[:, j].to(F64) * x[s]
        if bias is not None:
            out[t] += bias.to(F64)
    return out


# ---------------------------------------------------------------------------
# mixers (h: [T, width], one sequence from position 0)
# ---------------------------------------------------------------------------
def rglru(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
    T = h.shape[0]
    C, nb = int(m["width"]), int(m["blocks"])
    h = h.to(F64)
    gate = gelu_tanh(h @ w[p + "y"].to(F64).T + w[p + "y.b"].to(F64))
    c = causal_conv(h @ w[p + "x"].to(F64).T + w[p + "x.b"].to(F64), w[p + "conv"], w[p + "conv.b"])
    bs = C // nb
    r = torch.zeros(T, C, dtype=F64)
    i = torch.zeros(T, C, dtype=F64)
    for b in range(nb):
        cb = c[:, b * bs:(b + 1) * bs]
        r[:, b * bs:(b + 1) * bs] = sigmoid(cb @ w[p + "ra"][b].to(F64).T + w[p + "ra.b"][b].to(F64))
        i[:, b * bs:(b + 1) * bs] = sigmoid(cb @ w[p + "ri"][b].to(F64).T + w[p + "ri.b"][b].to(F64))
    a = torch.exp(-8.0 * r * softplus(w[p + "lam"].to(F64)))
    S = torch.zeros(C, dtype=F64)
    out = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1.0 - a[t] ** 2) * (i[t] * c[t])
        out[t] = S * gate[t]
    return out @ w[p + "o"].to(F64).T


def distance_bucket(d: int, rows: int, far: float) -> int:
    half = rows // 2
    if d < half:
        return d
    return min(rows - 1, half + int(math.floor(math.log(d / half) / math.log(far / half) * (rows - half))))


def attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, dim, vd = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    scale, cap, far = float(m["scale"]), m.get("softcap"), m.get("bias_max")          # cap and table are each optional
    h = h.to(F64)
    q = (h @ w[p + "q"].to(F64).T + w[p + "q.b"].to(F64)).view(T, H, dim)
    k = (h @ w[p + "k"].to(F64).T + w[p + "k.b"].to(F64)).view(T, G, dim)
    v = (h @ w[p + "v"].to(F64).T + w[p + "v.b"].to(F64)).view(T, G, vd)
    q = plain_norm(q, w[p + "q.norm"], eps)
    k = plain_norm(k, w[p + "k.norm"], eps)
    table = w[p + "rel"].to(F64) if far else None
    out = torch.zeros(T, H, vd, dtype=F64)
    for t in range(T):
        if far:
            bias = torch.stack([table[distance_bucket(t - j, table.shape[0], float(far))] for j in range(t + 1)])      # [t + 1, H]
        for hh in range(H):
            g = hh // (H // G)
            s = (k[:t + 1, g] @ q[t, hh]) * scale
            if cap:
                s = float(cap) * torch.tanh(s / float(cap))
            if far:
                s = s + bias[:, hh]
            e = torch.exp(s - s.max())
            out[t, hh] = (e / e.sum()) @ v[:t + 1, g]
    return out.reshape(T, H * vd) @ w[p + "o"].to(F64).T + w[p + "o.b"].to(F64)


def channel_delta(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, dim, vd = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    h = h.to(F64)
    q = silu(causal_conv(h @ w[p + "q"].to(F64).T, w[p + "q.conv"])).view(T, G, dim)
    k = silu(causal_conv(h @ w[p + "k"].to(F64).T, w[p + "k.conv"])).view(T, G, dim)
    v = silu(causal_conv(h @ w[p + "v"].to(F64).T, w[p + "v.conv"])).view(T, H, vd)
    q = q / torch.sqrt((q * q).sum(dim=-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    beta = sigmoid(h @ w[p + "b"].to(F64).T)                                                   # [T, H]
    low = h @ w[p + "a1"].to(F64).T
    g = torch.exp(-torch.exp(w[p + "A_log"].to(F64)).view(1, H, 1)
                  * softplus(low @ w[p + "a2"].to(F64).T + w[p + "dt_bias"].to(F64)).view(T, H, dim))
    out_gate = sigmoid((h @ w[p + "g1"].to(F64).T) @ w[p + "g2"].to(F64).T).view(T, H, vd)
    S = torch.zeros(H, dim, vd, dtype=F64)
    o = torch.zeros(T, H, vd, dtype=F64)
    for t in range(T):
        for hh in range(H):
            j = hh // (H // G)
            S[hh] = g[t, hh].view(dim, 1) * S[hh]
            e = beta[t, hh] * (v[t, hh] - S[hh].T @ k[t, j])
            S[hh] = S[hh] + torch.outer(k[t, j], e)
            o[t, hh] = S[hh].T @ q[t, j]
    o = plain_norm(o, w[p + "norm"], eps) * out_gate
    return o.reshape(T, H * vd) @ w[p + "o"].to(F64).T


# ---------------------------------------------------------------------------
# feed-forward
# ---------------------------------------------------------------------------
def relu2_expert(x: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    u = torch.clamp(x.to(F64) @ w[p + "up"].to(F64).T, min=0.0)
    return (u * u) @ w[p + "down"].to(F64).T


def routed_experts(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, f: dict) -> torch.Tensor:
    h = h.to(F64)
    top = int(f["router"]["top"])
    s = sigmoid(h @ w[p + "router"].to(F64).T)                # [T, experts]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in torch.topk(s[t], top).indices.tolist():
            out[t] += relu2_expert(s[t, e] * h[t:t + 1], w, f"{p}e{e}.")[0]
    if f.get("shared") is not None:
        out = out + sigmoid(h @ w[p + "shared.sg"].to(F64).T) * relu2_expert(h, w, p + "shared.")
    return out


# ---------------------------------------------------------------------------
# streams
# ---------------------------------------------------------------------------
def read_streams(X: Sequence[torch.Tensor], a: torch.Tensor) -> torch.Tensor:
    return sum(a[i].to(F64) * X[i].to(F64) for i in range(len(X)))


def write_streams(X: Sequence[torch.Tensor], M: torch.Tensor, b: torch.Tensor, y: torch.Tensor) -> List[torch.Tensor]:
    n = len(X)
    return [sum(M[i, j].to(F64) * X[i].to(F64) for i in range(n)) + b[j].to(F64) * y.to(F64) for j in range(n)]


# ---------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------
def run_order(cfg: dict) -> List[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


MIXERS = {"rglru": lambda n, w, p, m, eps: rglru(n, w, p, m), "attention": attention, "channel_delta": channel_delta}


def forward(w: Dict[str, torch.Tensor], cfg: dict, ids: Sequence[int], keep_layers: bool = False):
    """logits [T, vocab] in float64 (and, when asked, the sum of the streams after every layer run)."""
    eps = float(cfg["norm"]["eps"])
    n = int(cfg.get("streams", 1))
    hyper = "streams" in cfg
    x0 = w["embed"].to(F64)[list(ids)]
    X = [x0.clone() for _ in range(n)]
    sums = []
    for layer in run_order(cfg):
        L = cfg["layers"][layer]
        p = f"l{layer}."
        for q, kind in ((1, "mixer"), (2, "mlp")):
            if kind == "mlp" and L.get("mlp") is None:
                continue
            if hyper:
                a, M, b = (w[f"{p}hc{q}.{s}"].to(F64) for s in ("in", "mix", "out"))
            else:
                a, M, b = torch.ones(1, dtype=F64), torch.ones(1, 1, dtype=F64), torch.ones(1, dtype=F64)
            z = one_plus_norm(read_streams(X, a), w[f"{p}norm{q}"], eps)
            if kind == "mixer":
                y = MIXERS[L["type"]](z, w, p + "mix.", L["mixer"], eps)
            else:
                y = routed_experts(z, w, p + "mlp.", L["mlp"])
            y = y * w[f"{p}ls{q}"].to(F64)
            X = write_streams(X, M, b, y)
        sums.append(sum(X).clone())
    x = sum(X)
    logits = one_plus_norm(x, w["final.norm"], eps) @ w["head"].to(F64).T
    return (logits, torch.stack(sums)) if keep_layers else logits
