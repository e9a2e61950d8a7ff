"""Small Kadodra configurations for the tests, each unlike the others in every size and option, and helpers to
write a model folder with random weights and to read it back for the plain implementation."""
from __future__ import annotations

import copy

import torch


def _latent(heads, dim, rot_dim, vdim, rank, scale, window=None, base=1e4, scaling=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if rot_dim:
        m["rot"] = {"base": base, "dims": rot_dim}
        if scaling:
            m["rot"]["scaling"] = scaling
    if window:
        m["mask"] = {"size": window}
    return m


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


CASES = {
    # lightning first; a loop over the two middle layers, three passes; a layer without a feed-forward;
    # two experts per token; one latent layer with a window and stretched rotation, one without either
    "P": {
        "architecture": "Kadodra", "vocab": 200, "width": 64, "logit_scale": 0.5, "norm": {"eps": 1e-5},
        "loop": {"start": 1, "stop": 3, "times": 3},
        "layers": [
            {"type": "lightning", "mixer": {"heads": 3, "dim": 16, "vdim": 24, "decay": [0.9, 0.5, 1.0]}, "mlp": _dense(96)},
            {"type": "latent_attention", "mlp": _moe(5, 2, 40, 1.5),
             "mixer": _latent(4, 16, 8, 20, 24, 0.2, window=40, base=1e4,
                              scaling={"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0})},
            {"type": "lightning", "mixer": {"heads": 1, "dim": 40, "vdim": 72, "decay": [0.97]}, "mlp": None},
            {"type": "latent_attention", "mixer": _latent(2, 8, 16, 8, 40, 0.35), "mlp": _dense(48)},
        ],
    },
    # no loop; a window of exactly one page (a ring without slack); one expert per token; heads that are no
    # power of two; a latent wider than the heads
    "Q": {
        "architecture": "Kadodra", "vocab": 310, "width": 96, "logit_scale": 2.0, "norm": {"eps": 1e-6},
        "layers": [
            {"type": "latent_attention", "mlp": _moe(3, 1, 56, 3.0),
             "mixer": _latent(5, 24, 8, 12, 48, 0.18, window=64, base=5e4)},
            {"type": "lightning", "mixer": {"heads": 2, "dim": 24, "vdim": 40, "decay": [0.999, 0.7]}, "mlp": _dense(80)},
            {"type": "latent_attention", "mlp": None,
             "mixer": _latent(3, 12, 4, 28, 20, 0.3, window=7, base=1e3,
                              scaling={"factor": 2.5, "original": 32, "fast": 4.0, "slow": 1.0})},
        ],
    },
    # the loop covers everything, twice; three experts per token out of four; no rotated part at all in one layer
    "R": {
        "architecture": "Kadodra", "vocab": 150, "width": 48, "logit_scale": 1.0, "norm": {"eps": 3e-6},
        "loop": {"start": 0, "stop": 2, "times": 2},
        "layers": [
            {"type": "latent_attention", "mlp": _moe(4, 3, 24, 0.8), "mixer": _latent(2, 12, 0, 16, 16, 0.25, window=33)},
            {"type": "lightning", "mixer": {"heads": 4, "dim": 8, "vdim": 8, "decay": [0.3, 0.6, 0.9, 0.99]}, "mlp": _dense(64)},
        ],
    },
}
SEEDS = {"P": 5, "Q": 6, "R": 7}


def case(name: str) -> dict:
    return copy.deepcopy(CASES[name])


def write_folder(name: str, path: str, sink_boost: float = 0.0) -> str:
    from toyinfer_b200.weights import write_model_folder
    write_model_folder(case(name), SEEDS[name], path)
    return path


def read_folder(path: str):
    """(weights by name, config dict) for the plain implementation, through its own reader."""
    from plain.qwen3_plain import read_config, read_weights
    return read_weights(path), read_config(path)


def prompts(name: str, lengths, seed: int = 0):
    g = torch.Generator().manual_seed(4000 + seed)
    v = CASES[name]["vocab"]
    return [torch.randint(0, v, (n,), generator=g).tolist() for n in lengths]


def assert_close_logits(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "") -> None:
    """float32 engine: 2e-5 + 2e-4 |want| against the float64 result: the sharp test.  bfloat16 engine: every
    projection's output is rounded to 2^-9 relative, some ten roundings a layer run over up to eight runs, and the final
    norm carries the stream's error into logits whose spread is small in these random models: a row's error (mean
    taken off, root mean square) is a few hundredths of the row's spread as a rule and up to 0.12 now and then; the bound is
    a fifth, and half the spread for single logits.  (The same code runs in both types: what the float32 run passes is right.)"""
    got, want = got.detach().cpu().double(), want.detach().cpu().double()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert torch.isfinite(got).all(), what
    if dtype == "float32":
        torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-5, msg=lambda m: f"{what}: {m}")
    else:
        spread = want.std(dim=-1, keepdim=True) + 1e-3
        bad = (got - want).abs() > 0.5 * spread + 0.03 * want.abs()
        assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.numel()} logits off, worst {(got - want).abs().max():.4g}"
        err = (got - want - (got - want).mean(dim=-1, keepdim=True)).pow(2).mean(dim=-1).sqrt() / spread.squeeze(-1)
        assert err.max() < 0.2, f"{what}: a row is off by {err.max():.3g} of its spread"
