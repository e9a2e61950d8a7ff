"""Tusasun's mechanisms one at a time against the plain implementation (tests/plain/tusasun_plain.py): the residual
streams and their norm, the short convolution and its state, the recurrent block, attention with soft cap and
distance table (bucket edges and far keys made to stand out), the gated delta rule (long decoding), and the scored
experts (both ways the grouped products run).  Mixers run as prompts, single tokens, pieces of several sizes and
unequal batches, in slots that were used before."""
from __future__ import annotations

import pytest
import torch

from plain import tusasun_plain as plain
from test_kadodra_parts_gpu import DEV, DT, batch_for, bind_random, ctx_for, tol

pytestmark = pytest.mark.gpu


# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("S,H", [(1, 40), (3, 300), (4, 72), (8, 1100)])
def test_streams_update_read_and_norm(dtype, S, H):
    from toyinfer_b200.kernels import hyper
    g = torch.Generator().manual_seed(S)
    M = 7
    X = torch.randn(M, S, H, generator=g) * 3
    y = torch.randn(M, H, generator=g).to(dtype)
    gain = torch.rand(H, generator=g) + 0.5
    carry = torch.randn(S, S, generator=g)
    write, read = torch.randn(S, generator=g), torch.randn(S, generator=g)
    w = torch.randn(H, generator=g) * 0.1
    Xs = [X[:, s].double() for s in range(S)]
    new = plain.write_streams(Xs, carry, write, y.double() * gain.double())
    dev = lambda t: t.to(DEV)
    # a pending update and a read
    Xd = X.reshape(M, S * H).to(DEV).clone()
    pend = hyper.StreamUpdate(dev(y), dev(gain), dev(carry), dev(write))
    out = hyper.hyper_norm(Xd, pend, dev(read), dev(1.0 + w), 1e-5, dtype, S)
    torch.testing.assert_close(Xd.cpu().view(M, S, H).double(), torch.stack(new, dim=1), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(out.cpu().double(), plain.one_plus_norm(plain.read_streams(new, read), w, 1e-5), **tol(dtype, 3.0))
    # nothing pending, identity defaults: the sum of the streams
    Xd = X.reshape(M, S * H).to(DEV).clone()
    out, total = hyper.hyper_norm(Xd, None, None, dev(1.0 + w), 1e-5, dtype, S, want_sum=True)
    torch.testing.assert_close(total.cpu().double(), sum(Xs), rtol=1e-5, atol=1e-5)
    assert torch.equal(Xd.cpu(), X.reshape(M, S * H))
    # gathered rows with a pending update: the streams are left alone
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    out = hyper.hyper_norm(Xd, pend, None, dev(1.0 + w), 1e-5, dtype, S, rows=rows)
    torch.testing.assert_close(out.cpu().double(), plain.one_plus_norm(sum(new), w, 1e-5)[[5, 0, 5]], **tol(dtype, 3.0))
    assert torch.equal(Xd.cpu(), X.reshape(M, S * H))


def test_embedding_rows_several_times_over():
    from toyinfer_b200.kernels import wide
    table = torch.randn(30, 24).to(torch.bfloat16)
    ids = torch.tensor([3, 29, 0, 3], dtype=torch.int32)
    out = wide.embed_wide(table.to(DEV), ids.to(DEV), 1.0, 3).cpu()
    assert out.shape == (4, 72)
    for c in range(3):
        assert torch.equal(out[:, 24 * c:24 * (c + 1)], table.float()[ids.long()])


# ---------------------------------------------------------------------------
def feed(mixer, request, xs, schedule, dtype, n_slots=4, pre_use=True):
    """Runs sequences ``xs`` (inputs [T, hidden] each) through ``mixer`` as ``schedule`` says: a list of steps, each a list
    of (sequence, new tokens).  The slots were used by another sequence before when ``pre_use``.  Returns every
    sequence's outputs in order."""
    from toyinfer_b200.cache import CacheManager
    cache = CacheManager([request], 64 * 40, n_slots, 1024, dtype, DEV)
    if pre_use:                       # dirty every slot and page, then give them back
        hidden = xs[0].shape[1]
        junk = [cache.allocate_slot() for _ in range(n_slots)]
        for s in junk:
            cache.reserve(s, 130)
        cache.flush()
        x = (torch.randn(130 * n_slots, hidden, generator=torch.Generator().manual_seed(99)) * 2).to(dtype).to(DEV)
        mixer.forward(x, batch_for("start", junk, [0] * n_slots, [130] * n_slots, cache.scratch_slot), cache.view(0), {})
        for s in junk:
            cache.release(s)
    slots = {}
    fed = {i: 0 for i in range(len(xs))}
    outs = {i: [] for i in range(len(xs))}
    for step in schedule:
        who = [i for i, _ in step]
        news = [n for _, n in step]
        for i in who:
            if i not in slots:
                slots[i] = cache.allocate_slot()
        starts = [fed[i] for i in who]
        for i, st, nw in zip(who, starts, news):
            cache.reserve(slots[i], st + nw)
        cache.flush()
        mode = "start" if all(st == 0 for st in starts) else "extend" if all(nw == 1 for nw in news) else "mixed"
        x = torch.cat([xs[i][st:st + nw] for i, st, nw in zip(who, starts, news)]).to(DEV)
        got = mixer.forward(x, batch_for(mode, [slots[i] for i in who], starts, news, cache.scratch_slot), cache.view(0), {}).cpu().double()
        o = 0
        for i, st, nw in zip(who, starts, news):
            outs[i].append(got[o:o + nw])
            o += nw
            cache.commit(slots[i], st + nw)
            fed[i] = st + nw
    return [torch.cat(outs[i]) for i in range(len(xs))]


def schedules(lens):
    """Three ways to feed sequences of these lengths: all at once; a prompt then single tokens; pieces of unequal sizes
    down to two tokens, the sequences side by side."""
    whole = [[(i, n) for i, n in enumerate(lens)]]
    heads = [max(1, n - 40 - 7 * i) for i, n in enumerate(lens)]
    decode = [[(i, h) for i, h in enumerate(heads)]]
    for t in range(max(n - h for n, h in zip(lens, heads))):
        decode.append([(i, 1) for i, (n, h) in enumerate(zip(lens, heads)) if h + t < n])
    sizes = [[2, 61, 3, 70, 1, 64, 2], [64, 2, 1, 1, 63], [1, 2, 2, 130]]
    pieces, fed, k = [], [0] * len(lens), 0
    while any(f < n for f, n in zip(fed, lens)):
        step = []
        for i, n in enumerate(lens):
            if fed[i] < n:
                want = sizes[i % 3][k] if k < len(sizes[i % 3]) else n
                take = min(want, n - fed[i])
                step.append((i, take))
                fed[i] += take
        pieces.append(step)
        k += 1
    return {"whole": whole, "decode": decode, "pieces": pieces}


def check_all_schedules(mixer, xs, wants, dtype, scale=3.0):
    lens = [x.shape[0] for x in xs]
    for name, sch in schedules(lens).items():
        got = feed(mixer, mixer.memory_request(), xs, sch, dtype)
        for i, (g, w) in enumerate(zip(got, wants)):
            torch.testing.assert_close(g, w, **tol(dtype, scale), msg=lambda e: f"{name}, sequence {i}: {e}")


def inputs(lens, hidden, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(n, hidden, generator=g) * 1.5).to(dtype) for n in lens]


# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("taps,C", [(1, 40), (2, 200), (4, 130), (7, 24)])
def test_short_convolution_and_its_state(dtype, taps, C):
    """The kernel alone, with both biases and silu, through pieces that are shorter than the filter, chunks of 64 and longer runs."""
    from toyinfer_b200.cache import CacheManager
    from toyinfer_b200.engine.batch import BatchBuffers, fill_batch
    from toyinfer_b200.kernels import recurrent as KR
    from toyinfer_b200.parts import StateRequest
    g = torch.Generator().manual_seed(taps)
    T = 300
    x = torch.randn(T, C + 8, generator=g).to(dtype)                    # the channels are columns 8 .. of a wider row
    w = torch.randn(C, taps, generator=g)
    ib, ob = torch.randn(C, generator=g), torch.randn(C, generator=g)
    want = plain.silu(plain.causal_conv(x[:, 8:].double() + ib.double(), w, ob))
    cache = CacheManager([StateRequest((5 + max(taps - 1, 1) * C,), torch.float32)], 64, 2, 1024, dtype, DEV)
    cache.allocate_slot()
    s = cache.allocate_slot()
    state = cache.view(0).state
    state[s] = 0
    fed, got = 0, []
    for n in [1, 1, 2, 3, 64, 65, 1, 130, 2, T]:
        n = min(n, T - fed)
        if n <= 0:
            break
        b = batch_for("start" if fed == 0 else "extend" if n == 1 else "mixed", [s], [fed], [n], cache.scratch_slot)
        got.append(KR.short_conv(x[fed:fed + n, 8:].to(DEV), w.to(DEV), state, 5, b, in_bias=ib.to(DEV), out_bias=ob.to(DEV), act="silu").cpu())
        fed += n
    torch.testing.assert_close(torch.cat(got).double(), want, **tol(dtype, 3.0))


RGLRU = [dict(width=96, blocks=3, conv=4), dict(width=40, blocks=1, conv=1), dict(width=130, blocks=5, conv=2), dict(width=256, blocks=2, conv=3)]


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("chunked_from", [None, 2])
@pytest.mark.parametrize("c", RGLRU)
def test_recurrent_block(dtype, c, chunked_from, monkeypatch):
    """``chunked_from``: every step that brings a sequence two tokens or more runs the chunked form of the recurrence (chunks
    of 128 in parallel, a walk over their effects), which otherwise starts at 256."""
    from toyinfer_b200.kernels import recurrent as KR
    from toyinfer_b200.parts import PartSpec, build_part
    if chunked_from is not None:
        monkeypatch.setattr(KR, "RGLRU_CHUNKED_FROM", chunked_from)
    hidden = 56
    m = build_part("mixer", PartSpec("rglru", dict(c)), ctx_for(dtype, hidden), "a.")

    def edit(cpu):                  # decays from nearly none to nearly all, so that a lost or doubled state shows
        cpu["a.lam"].copy_(torch.linspace(-6.0, 2.0, c["width"]))
    w = bind_random(m, 3, dtype, edit)
    xs = inputs([300, 129, 3], hidden, 5, dtype)
    wants = [plain.rglru(x.double(), w, "a.", c) for x in xs]
    check_all_schedules(m, xs, wants, dtype)


ATT = [dict(n_heads=4, n_kv_heads=2, dim=24, vdim=40, softcap=30.0, bias_rows=12, bias_max=50.0),
       dict(n_heads=3, n_kv_heads=3, dim=64, vdim=16, softcap=1.5, bias_rows=32, bias_max=400.0),
       dict(n_heads=6, n_kv_heads=1, dim=8, vdim=8, softcap=0.0, bias_rows=0, bias_max=0.0),
       dict(n_heads=2, n_kv_heads=1, dim=128, vdim=200, softcap=50.0, bias_rows=6, bias_max=9.0),
       # the two shapes that the tensor-core kernel takes in bfloat16 (keys and values of 64 or of 128)
       dict(n_heads=4, n_kv_heads=2, dim=64, vdim=64, softcap=20.0, bias_rows=16, bias_max=100.0),
       dict(n_heads=2, n_kv_heads=1, dim=128, vdim=128, softcap=0.0, bias_rows=8, bias_max=300.0),
       dict(n_heads=2, n_kv_heads=2, dim=128, vdim=128, softcap=3.0, bias_rows=0, bias_max=0.0)]


def att_cfg(c, scale):
    m = {"heads": c["n_heads"], "kv_heads": c["n_kv_heads"], "dim": c["dim"], "vdim": c["vdim"], "scale": scale}
    if c["softcap"]:
        m["softcap"] = c["softcap"]
    if c["bias_max"]:
        m["bias_max"] = c["bias_max"]
    return m


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("c", ATT)
def test_attention_with_cap_and_distance_table(dtype, c):
    """The table's rows differ by several units from one to the next, so that a key put into a neighbour's bucket (one
    position off at an edge) changes the weights visibly; prompts are longer than the table's reach and than a page."""
    from toyinfer_b200.parts import PartSpec, build_part
    hidden, scale = 56, 0.4
    m = build_part("mixer", PartSpec("biased_attention", dict(c, scale=scale, eps=1e-5)), ctx_for(dtype, hidden), "a.")

    def edit(cpu):
        if "a.rel" in cpu:
            cpu["a.rel"].mul_(3.0)
    w = bind_random(m, 4, dtype, edit)
    xs = inputs([203, 131, 2], hidden, 6, dtype)
    wants = [plain.attention(x.double(), w, "a.", att_cfg(c, scale), 1e-5) for x in xs]
    check_all_schedules(m, xs, wants, dtype)


@pytest.mark.parametrize("dtype", DT)
def test_attention_finds_one_far_key(dtype):
    """The table favours the furthest bucket of head 0 by 12 units and the nearest of head 1: head 0 of a late query
    looks at the oldest keys, hundreds of positions and several pages back, head 1 at itself; single tokens after the
    prompt keep doing so while the buckets' edges pass over the old keys."""
    from toyinfer_b200.parts import PartSpec, build_part
    hidden = 40
    c = dict(n_heads=2, n_kv_heads=2, dim=16, vdim=16, softcap=5.0, bias_rows=10, bias_max=600.0)
    m = build_part("mixer", PartSpec("biased_attention", dict(c, scale=0.3, eps=1e-5)), ctx_for(dtype, hidden), "a.")

    def edit(cpu):
        cpu["a.rel"].zero_()
        cpu["a.rel"][-1, 0] = 12.0
        cpu["a.rel"][0, 1] = 12.0
    w = bind_random(m, 8, dtype, edit)
    xs = inputs([700], hidden, 9, dtype)
    want = plain.attention(xs[0].double(), w, "a.", att_cfg(c, 0.3), 1e-5)
    sch = [[(0, 640)]] + [[(0, 1)]] * 60
    got = feed(m, m.memory_request(), xs, sch, dtype)[0]
    torch.testing.assert_close(got, want, **tol(dtype, 3.0))


DELTA = [dict(n_heads=4, n_qk_heads=2, dim=16, vdim=24, conv=4), dict(n_heads=2, n_qk_heads=2, dim=40, vdim=72, conv=2),
         dict(n_heads=3, n_qk_heads=1, dim=128, vdim=8, conv=3), dict(n_heads=1, n_qk_heads=1, dim=64, vdim=150, conv=1)]


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("c", DELTA)
def test_gated_delta_rule(dtype, c):
    from toyinfer_b200.parts import PartSpec, build_part
    hidden = 48
    m = build_part("mixer", PartSpec("channel_delta", dict(c, eps=1e-5, decay_rank=8, gate_rank=24)), ctx_for(dtype, hidden), "a.")

    def edit(cpu):                  # decays near one: what was written hundreds of tokens ago still counts
        cpu["a.dt_bias"].sub_(4.0)
    w = bind_random(m, 5, dtype, edit)
    xs = inputs([180, 70, 2], hidden, 7, dtype)
    cfg = {"heads": c["n_heads"], "kv_heads": c["n_qk_heads"], "dim": c["dim"], "vdim": c["vdim"], "conv": c["conv"]}
    wants = [plain.channel_delta(x.double(), w, "a.", cfg, 1e-5) for x in xs]
    check_all_schedules(m, xs, wants, dtype)


@pytest.mark.parametrize("dtype", DT)
def test_gated_delta_rule_decodes_for_long(dtype):
    from toyinfer_b200.parts import PartSpec, build_part
    hidden = 32
    c = dict(n_heads=2, n_qk_heads=1, dim=32, vdim=32, conv=4)
    m = build_part("mixer", PartSpec("channel_delta", dict(c, eps=1e-5)), ctx_for(dtype, hidden), "a.")
    w = bind_random(m, 6, dtype, lambda cpu: cpu["a.dt_bias"].sub_(5.0))
    xs = inputs([400], hidden, 8, dtype)
    cfg = {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "conv": 4}
    want = plain.channel_delta(xs[0].double(), w, "a.", cfg, 1e-5)
    got = feed(m, m.memory_request(), xs, [[(0, 5)]] + [[(0, 1)]] * 395, dtype)[0]
    torch.testing.assert_close(got, want, **tol(dtype, 3.0))


# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("experts,top,M,shared", [(5, 2, 70, 24), (3, 1, 1, 0), (4, 4, 9, 40), (16, 1, 200, 16), (2, 2, 130, 0),
                                                   (3, 1, 400, 8), (20, 6, 33, 0)])
@pytest.mark.parametrize("hidden,ff", [(40, 36), (136, 200)])
def test_scored_experts(dtype, experts, top, M, shared, hidden, ff):
    from toyinfer_b200.parts import PartSpec, build_part
    m = build_part("feed_forward", PartSpec("scored_moe", {"n_experts": experts, "top": top, "intermediate_size": ff,
                                                             "shared_size": shared}), ctx_for(dtype, hidden), "f.")

    def edit(cpu):                  # scores apart from one another and from one half, but not so large that two sigmoids are both 1
        cpu["f.router"].mul_(3.0)
    w = bind_random(m, 11, dtype, edit)
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, hidden, generator=g).to(dtype)
    f = {"router": {"experts": experts, "top": top}, "shared": {"ff": shared} if shared else None}
    # tokens whose top-th and next scores nearly tie are left out of the comparison
    z = x.double() @ w["f.router"].double().T
    srt = z.sort(dim=-1, descending=True).values
    clear = torch.ones(M, dtype=torch.bool) if top == experts else (srt[:, top - 1] - srt[:, top]) > 0.05
    assert clear.sum() >= M * 0.6
    want = plain.routed_experts(x.double(), w, "f.", f)
    got = m.forward(x.to(DEV), None).cpu().double()
    torch.testing.assert_close(got[clear], want[clear], **tol(dtype, 2.0))
