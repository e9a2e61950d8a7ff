"""Small Tusasun configurations for the tests, each unlike the others in every size and option, and helpers to write a
model folder with random weights and to read it back for the plain implementation."""
from __future__ import annotations

import copy

import torch


def _moe(experts, top, ff, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def _att(heads, kv, dim, vdim, scale, softcap=None, bias_max=None, bias_rows=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap:
        m["softcap"] = softcap
    if bias_max:
        m["bias_max"] = bias_max
        m["bias_rows"] = bias_rows
    return m


CASES = {
    # four streams; attention first, grouped (6 heads over 2), values wider than keys, a table of 12 rows that ends at 50;
    # a loop over the two middle layers, three passes; a layer without a feed-forward; two experts per token, no shared one
    "P": {
        "architecture": "Tusasun", "vocab": 210, "width": 64, "norm": {"eps": 1e-5}, "streams": 4,
        "loop": {"start": 1, "stop": 3, "times": 3},
        "layers": [
            {"type": "attention", "mixer": _att(6, 2, 16, 24, 0.25, softcap=30.0, bias_max=50, bias_rows=12), "mlp": _moe(5, 2, 40)},
            {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "conv": 3, "decay_rank": 8, "gate_rank": 16},
             "mlp": None},
            {"type": "rglru", "mixer": {"width": 96, "blocks": 3, "conv": 4}, "mlp": _moe(3, 1, 56, shared=24)},
            {"type": "attention", "mixer": _att(2, 2, 40, 8, 0.1, bias_max=300, bias_rows=32), "mlp": _moe(4, 4, 16, shared=72)},
        ],
    },
    # two streams, no loop; one query/key head for three value heads; a convolution of two taps and one of one tap (none);
    # attention without table or cap; a single gate block
    "Q": {
        "architecture": "Tusasun", "vocab": 310, "width": 96, "norm": {"eps": 1e-6}, "streams": 2,
        "layers": [
            {"type": "channel_delta", "mixer": {"heads": 3, "kv_heads": 1, "dim": 40, "vdim": 72, "conv": 2}, "mlp": _moe(6, 3, 24, shared=40)},
            {"type": "rglru", "mixer": {"width": 40, "blocks": 1, "conv": 1}, "mlp": _moe(2, 1, 80)},
            {"type": "attention", "mixer": _att(5, 1, 24, 12, 0.3), "mlp": None},
            {"type": "rglru", "mixer": {"width": 130, "blocks": 5, "conv": 2}, "mlp": _moe(9, 2, 32, shared=8)},
        ],
    },
    # one plain stream (no "streams" key: no connection tensors); the loop covers everything, twice; a soft cap low enough to bite
    "R": {
        "architecture": "Tusasun", "vocab": 150, "width": 48, "norm": {"eps": 3e-6},
        "loop": {"start": 0, "stop": 2, "times": 2},
        "layers": [
            {"type": "attention", "mixer": _att(3, 3, 12, 20, 0.5, softcap=2.0, bias_max=9, bias_rows=6), "mlp": _moe(4, 3, 24, shared=32)},
            {"type": "channel_delta", "mixer": {"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 8, "conv": 5}, "mlp": _moe(3, 2, 64)},
        ],
    },
    # a single stream WITH connection tensors; heads of 128 query/key elements in the delta rule
    "S": {
        "architecture": "Tusasun", "vocab": 120, "width": 40, "norm": {"eps": 1e-5}, "streams": 1,
        "layers": [
            {"type": "rglru", "mixer": {"width": 24, "blocks": 2, "conv": 3}, "mlp": _moe(2, 2, 16)},
            {"type": "channel_delta", "mixer": {"heads": 2, "kv_heads": 1, "dim": 128, "vdim": 16, "conv": 4}, "mlp": _moe(3, 1, 24, shared=16)},
        ],
    },
}
SEEDS = {"P": 15, "Q": 16, "R": 17, "S": 18}


def case(name: str) -> dict:
    return copy.deepcopy(CASES[name])


def write_folder(name: str, path: str) -> str:
    from toyinfer_b200.weights import write_model_folder
    write_model_folder(case(name), SEEDS[name], path)
    return path


def read_folder(path: str):
    """(weights by name, config dict) for the plain implementation, through its own reader."""
    from plain.qwen3_plain import read_config, read_weights
    return read_weights(path), read_config(path)


def prompts(name: str, lengths, seed: int = 0):
    g = torch.Generator().manual_seed(7000 + seed)
    v = CASES[name]["vocab"]
    return [torch.randint(0, v, (n,), generator=g).tolist() for n in lengths]


def assert_close_logits(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "") -> None:
    """float32 engine: 2e-5 + 2e-4 |want| against the float64 result: the sharp test, row by row.  bfloat16 engine: a
    row's error is its root mean square over the vocabulary (mean taken off) as a fraction of the row's spread.  Rounding
    alone leaves a few hundredths.  But these random routers have close calls: where the bfloat16 scores of two experts
    fall the other way, that token runs another expert and its row is off by much more (later tokens feel it faintly
    through states and keys).  With two thousand choices in a test and a close call in one of a hundred, up to a
    tenth of the rows are such.  So the rows are judged together: half of them within 0.08, all but one in seven (or one)
    within 0.25, and none further off than a row's whole spread and a half.  (The same code runs in both types: what
    the float32 run passes is right.)"""
    got, want = got.detach().cpu().double(), want.detach().cpu().double()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert torch.isfinite(got).all(), what
    if dtype == "float32":
        torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-5, msg=lambda m: f"{what}: {m}")
        return
    spread = want.std(dim=-1) + 1e-3
    d = got - want
    err = (d - d.mean(dim=-1, keepdim=True)).pow(2).mean(dim=-1).sqrt() / spread
    n = err.numel()
    report = f"{what}: row errors median {err.median():.3g}, max {err.max():.3g}, {int((err > 0.25).sum())} of {n} over 0.25"
    assert err.median() < 0.08, report
    assert int((err > 0.25).sum()) <= max(1, n // 7), report
    assert err.max() < 1.5, report
