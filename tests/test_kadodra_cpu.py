"""Kadodra on the host: configuration, order of layers, rotation tables, parameter names, random tables."""
from __future__ import annotations

import math

import pytest
import torch

from kadodra_cases import CASES, case
from plain import kadodra_plain as plain


def _cfg(raw):
    from toyinfer_b200 import models  # noqa: F401
    from toyinfer_b200.config.registry import architecture_of
    arch = architecture_of(raw)
    return arch, arch.config_cls.from_dict(raw)


def test_the_design_is_found_by_its_name_and_reads_every_case():
    for name in CASES:
        arch, cfg = _cfg(case(name))
        assert arch.name == "Kadodra" and cfg.width == CASES[name]["width"]


@pytest.mark.parametrize("name", list(CASES))
def test_order_of_layers_matches_the_plain_reading(name):
    _, cfg = _cfg(case(name))
    assert cfg.run_order() == plain.run_order(case(name))


def test_order_with_a_loop_in_the_middle():
    raw = case("P")
    _, cfg = _cfg(raw)
    assert cfg.run_order() == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    raw["loop"] = {"start": 2, "stop": 2, "times": 4}          # an empty span
    assert _cfg(raw)[1].run_order() == [(i, False) for i in range(4)]


def test_bad_configurations_are_refused_with_all_their_faults():
    from toyinfer_b200.config import ConfigError
    raw = case("Q")
    raw["layers"][0]["mixer"]["rot"]["dims"] = 6
    raw["layers"][1]["mixer"]["decay"] = [0.5]
    raw["loop"] = {"start": 2, "stop": 1, "times": 1}
    del raw["norm"]["eps"]
    with pytest.raises(ConfigError) as e:
        _cfg(raw)
    msg = str(e.value)
    for part in ("rot.dims", "decay", "loop", "norm.eps"):
        assert part in msg, msg


def test_schedule_memory_and_names():
    from toyinfer_b200.parts.model import DecoderModel
    from toyinfer_b200.parts import KVRequest, StateRequest
    arch, cfg = _cfg(case("P"))
    m = DecoderModel(arch.describe(cfg), torch.float32, "cpu")
    assert [(e.layer, e.add_embedding) for e in m.schedule] == cfg.run_order()
    req = m.memory_requests()
    assert isinstance(req[0], StateRequest) and req[0].shape == (3, 16, 24)
    assert req[1] == KVRequest(1, 32, 40, values=False) and req[3] == req[1]      # every pass has memory of its own
    assert req[7] == KVRequest(1, 56, 0, values=False)
    names = set(m.param_specs())
    for n in ("embed", "final.norm", "l0.norm1", "l0.mix.g", "l0.mlp.up", "l1.mix.dkv.norm", "l1.mix.sink", "l1.mlp.e4.down",
              "l1.mlp.table", "l3.mix.uk"):
        assert n in names, n
    assert not any(n.startswith("l2.mlp") for n in names)


@pytest.mark.parametrize("scaling", [None, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0},
                                     {"factor": 1.0, "original": 4096, "fast": 32.0, "slow": 1.0},
                                     {"factor": 16.0, "original": 8, "fast": 1.0, "slow": 0.5}])
@pytest.mark.parametrize("dims,base", [(8, 1e4), (30, 5e5)])
def test_rotation_tables(dims, base, scaling):
    from toyinfer_b200.parts.rope import rotary_tables
    cos, sin = rotary_tables(dims, base, 300, scaling)
    freqs, mag = plain.scaled_frequencies(dims, base, scaling)
    for pos in (0, 1, 17, 299):
        for i in range(dims // 2):
            assert abs(float(cos[pos, i]) - math.cos(pos * freqs[i]) * mag) < 2e-6
            assert abs(float(sin[pos, i]) - math.sin(pos * freqs[i]) * mag) < 2e-6


def test_random_tables_have_different_experts_in_a_row():
    from toyinfer_b200.parts import ParamSpec
    from toyinfer_b200.weights.random_init import draw
    t = draw(ParamSpec((50, 3), role="int_table", init="distinct_below", high=4), "x.table", 1)
    assert t.dtype == torch.int32 and int(t.min()) >= 0 and int(t.max()) <= 3
    assert all(len(set(r.tolist())) == 3 for r in t)
    assert len({tuple(r.tolist()) for r in t}) > 5


def test_a_written_folder_reads_back_for_both_sides(tmp_path):
    from kadodra_cases import read_folder, write_folder
    w, cfg = read_folder(write_folder("R", str(tmp_path)))
    assert cfg["loop"]["times"] == 2 and w["l0.mlp.table"].shape == (150, 3)
    logits = plain.forward(w, cfg, [3, 1, 4, 1, 5])
    assert logits.shape == (5, 150) and torch.isfinite(logits).all()
