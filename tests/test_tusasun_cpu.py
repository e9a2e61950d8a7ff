"""What of the Tusasun design needs no device: the configuration's checks, the order layers run in, the distance
table's buckets, and tensors whose sizes the checkpoint decides."""
from __future__ import annotations

import pytest
import torch

from plain import tusasun_plain as plain
from tusasun_cases import CASES, case


def config(d):
    from toyinfer_b200 import models  # noqa: F401
    from toyinfer_b200.config.registry import architecture_of
    arch = architecture_of(d)
    return arch, arch.config_cls.from_dict(d)


@pytest.mark.parametrize("name", list(CASES))
def test_layers_run_in_the_plain_order_with_memory_per_pass(name):
    from toyinfer_b200.parts.model import DecoderModel
    arch, cfg = config(case(name))
    assert cfg.run_order() == plain.run_order(case(name))
    model = DecoderModel(arch.describe(cfg), torch.float32, "cpu")
    assert [e.layer for e in model.schedule] == plain.run_order(case(name))
    reqs = model.memory_requests()
    assert len(reqs) == len(model.schedule) and all(r is not None for r in reqs)          # every pass has memory of its own


def test_configuration_problems_are_all_reported():
    from toyinfer_b200.config.base import ConfigError
    d = case("P")
    d["streams"] = 9
    d["layers"][0]["mixer"]["kv_heads"] = 4                  # 6 heads over 4
    d["layers"][2]["mixer"]["blocks"] = 5                    # 96 channels in 5 blocks
    d["layers"][1]["type"] = "nothing"
    d["loop"]["stop"] = 7
    with pytest.raises(ConfigError) as e:
        config(d)
    msg = str(e.value)
    for piece in ("streams", "6 heads over 4", "96 channels", "layers[1].type", "loop"):
        assert piece in msg, (piece, msg)


def test_sizes_that_only_the_checkpoint_knows(tmp_path):
    """The rows of a distance table and the ranks of the delta rule's low-rank projections come with the tensors: a
    folder written with other ones than the description would draw loads, and the parts take the tensors' sizes."""
    from toyinfer_b200.parts.model import DecoderModel
    from toyinfer_b200.weights import load_parameters, write_model_folder
    d = case("P")
    d["layers"][0]["mixer"]["bias_rows"] = 20
    d["layers"][1]["mixer"]["decay_rank"] = 5
    d["layers"][1]["mixer"]["gate_rank"] = 11
    write_model_folder(d, 3, str(tmp_path))
    arch, cfg = config(case("P"))                            # described without knowing those sizes
    model = DecoderModel(arch.describe(cfg), torch.float32, "cpu")
    model.bind(load_parameters(model.param_specs(), str(tmp_path), torch.float32, "cpu"))
    att, delta = model.blocks[0].mixer, model.blocks[1].mixer
    assert att.bias_rows == 20 and att.dist_bias.shape == (6, 51)
    assert (delta.rank_a, delta.rank_g) == (5, 11)


def test_without_the_streams_key_there_are_no_connection_tensors():
    from toyinfer_b200.parts.model import DecoderModel
    arch, cfg = config(case("R"))
    names = DecoderModel(arch.describe(cfg), torch.float32, "cpu").param_specs()
    assert not any(".hc" in n for n in names) and "l0.ls1" in names
    arch, cfg = config(case("S"))                            # one stream, but named: the tensors are there
    names = DecoderModel(arch.describe(cfg), torch.float32, "cpu").param_specs()
    assert names["l0.hc1.mix"].shape == (1, 1)


def test_distance_buckets_follow_the_rule():
    from toyinfer_b200.parts.biased_attention import distance_buckets
    for rows, far in [(16, 120.0), (12, 50.0), (32, 400.0), (6, 9.0), (2, 5.0), (64, 1000.5)]:
        got = distance_buckets(rows, far).tolist()
        assert got == [plain.distance_bucket(d, rows, far) for d in range(len(got))]
        assert got[-1] == rows - 1                                       # the table's reach ends in its last row
        assert all(plain.distance_bucket(d, rows, far) == rows - 1 for d in range(len(got), len(got) + 2000, 37))
