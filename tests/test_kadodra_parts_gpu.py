"""Kadodra's mechanisms one at a time against the plain implementation (tests/plain/kadodra_plain.py): the float32
stream and its norm, latent attention with its cache (prompts, single tokens, pieces; a window's edge, sinks and
far keys made to stand out), lightning attention in its three forms, and the two feed-forwards."""
from __future__ import annotations

import pytest
import torch

from plain import kadodra_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"
DT = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    return dict(rtol=2e-4, atol=2e-5 * scale) if dtype == torch.float32 else dict(rtol=3e-2, atol=2e-2 * scale)


def ctx_for(dtype, hidden, positions=None):
    from toyinfer_b200.parts import BuildContext
    c = BuildContext(dtype=dtype, device=torch.device(DEV), hidden_size=hidden)
    c.positions.update(positions or {})
    return c


def bind_random(part, seed, dtype, edit=None):
    """Draws the part's tensors on the CPU, lets ``edit`` change them, binds device copies, returns the CPU ones
    (as the engine's type holds them)."""
    from toyinfer_b200.weights import random_parameters
    cpu = random_parameters(part.param_specs(), seed, torch.float32, "cpu")
    if edit:
        edit(cpu)
    if dtype == torch.bfloat16:
        cpu = {k: (v if v.dtype == torch.int32 else v.to(torch.bfloat16).float()) for k, v in cpu.items()}
    part.bind({k: (v.to(DEV) if v.dtype == torch.int32 else v.to(DEV, dtype)) for k, v in cpu.items()})
    return cpu


def batch_for(mode, slots, starts, news, scratch, ids=None):
    from toyinfer_b200.engine.batch import BatchBuffers, fill_batch
    buf = BatchBuffers(len(slots), sum(news), DEV)
    toks = ids if ids is not None else [[0] * n for n in news]
    return fill_batch(buf, mode, slots, starts, toks, scratch, 4096)


# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("H", [40, 300])
def test_float32_stream_and_its_norm(dtype, H):
    from toyinfer_b200.kernels import wide
    g = torch.Generator().manual_seed(1)
    h = torch.randn(9, H, generator=g) * 3
    ds = [torch.randn(9, H, generator=g).to(dtype) for _ in range(3)]
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(dtype)
    for n_terms in range(4):
        hd = h.to(DEV).clone()
        terms = tuple(d.to(DEV) for d in ds[:n_terms])
        y = wide.add_norm_wide(hd, terms if n_terms != 1 else terms[0], w.to(DEV), 1e-5, dtype)
        want = h.double()
        if n_terms >= 2:
            want = want + (ds[0].double() + ds[1].double())
        elif n_terms == 1:
            want = want + ds[0].double()
        if n_terms == 3:
            want = want + ds[2].double()
        torch.testing.assert_close(hd.cpu().double(), want, rtol=1e-6, atol=1e-6)       # the stream itself stays 32-bit
        torch.testing.assert_close(y.cpu().double(), plain.rms_norm(want, w.double(), 1e-5), **tol(dtype))
    # gathered rows: the stream is left alone
    hd = h.to(DEV).clone()
    rows = torch.tensor([7, 0, 7], dtype=torch.int32, device=DEV)
    y = wide.add_norm_wide(hd, (ds[0].to(DEV), ds[1].to(DEV)), w.to(DEV), 1e-5, dtype, rows=rows)
    want = plain.rms_norm(h.double() + (ds[0].double() + ds[1].double()), w.double(), 1e-5)[[7, 0, 7]]
    torch.testing.assert_close(y.cpu().double(), want, **tol(dtype))
    assert torch.equal(hd.cpu(), h)


def test_embedding_into_the_stream():
    from toyinfer_b200.kernels import wide
    table = torch.randn(30, 24).to(torch.bfloat16)
    ids = torch.tensor([3, 29, 0, 3], dtype=torch.int32)
    out = wide.embed_wide(table.to(DEV), ids.to(DEV))
    assert out.dtype == torch.float32 and torch.equal(out.cpu(), table.float()[ids.long()])


# ---------------------------------------------------------------------------
LATENT = [
    # heads, dim, rot, vdim, rank, window, scaling
    dict(heads=3, dim=8, rot=4, vdim=12, rank=20, window=0, scaling=None),
    dict(heads=5, dim=16, rot=8, vdim=8, rank=24, window=37, scaling={"factor": 3.0, "original": 50, "fast": 6.0, "slow": 1.5}),
    dict(heads=2, dim=4, rot=16, vdim=24, rank=70, window=64, scaling=None),
    dict(heads=34, dim=6, rot=2, vdim=5, rank=10, window=5, scaling=None),
    # heads that fill the tensor-core prompt kernel's 128 and 64 elements exactly, and ones that leave room
    dict(heads=2, dim=64, rot=64, vdim=128, rank=64, window=100, scaling=None),
    dict(heads=3, dim=32, rot=32, vdim=64, rank=32, window=0, scaling=None),
    dict(heads=2, dim=40, rot=32, vdim=72, rank=16, window=65, scaling={"factor": 2.0, "original": 40, "fast": 4.0, "slow": 1.0}),
    # more heads than one tensor-core tile of 16 rows holds, and more than two; latents of more than 128 and 256 elements
    dict(heads=20, dim=8, rot=8, vdim=8, rank=24, window=50, scaling=None),
    dict(heads=40, dim=8, rot=8, vdim=16, rank=40, window=0, scaling=None),
    dict(heads=3, dim=8, rot=24, vdim=8, rank=136, window=0, scaling=None),
    dict(heads=2, dim=8, rot=8, vdim=8, rank=264, window=70, scaling=None),
]


def make_latent(dtype, c, hidden=56, seed=3, edit=None):
    from toyinfer_b200.parts import PartSpec, build_part
    ctx = ctx_for(dtype, hidden)
    ctx.positions["r"] = build_part("position", PartSpec("rotary_half", {"dim": c["rot"], "theta": 3e3, "max_positions": 512,
                                                                         "scaling": c["scaling"]}), ctx, "")
    m = build_part("mixer", PartSpec("latent_attention", {
        "n_heads": c["heads"], "dim": c["dim"], "rot_dim": c["rot"], "vdim": c["vdim"], "kv_rank": c["rank"], "scale": 0.3,
        "eps": 1e-5, "position": "r", "window": c["window"]}), ctx, "a.")
    w = bind_random(m, seed, dtype, edit)
    mcfg = {"heads": c["heads"], "dim": c["dim"], "rot_dim": c["rot"], "vdim": c["vdim"], "kv_rank": c["rank"], "scale": 0.3,
            "rot": {"base": 3e3, "dims": c["rot"], "scaling": c["scaling"]}}
    if c["window"]:
        mcfg["mask"] = {"size": c["window"]}
    return m, w, mcfg


def loud_inputs(T, hidden, seed, loud=()):
    """Random rows; the rows at ``loud`` are 30 times larger: the rotated key part is not normed, so such a token's
    score stands out (one way or the other) for every query that sees it, and is gone the step after it leaves the window."""
    x = torch.randn(T, hidden, generator=torch.Generator().manual_seed(seed))
    for j in loud:
        x[j] *= 30.0
    return x


def sinks_that_matter(cpu):
    s = cpu["a.sink"]
    s[0] = 6.0            # takes most of head 0's weight
    s[1] = -30.0          # takes none of head 1's


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("c", LATENT)
def test_latent_attention_prompt_then_single_tokens(dtype, c):
    from toyinfer_b200.cache import CacheManager
    m, w, mcfg = make_latent(dtype, c, edit=sinks_that_matter)
    n, extra = 150, 70
    W = c["window"]
    loud = [3, 64, 127, 128, n - 1] + ([n - W, n - W + 1] if W else [])
    x = loud_inputs(n + extra, 56, 7, loud).to(dtype)
    want = plain.latent_attention(x.double(), w, "a.", mcfg, 1e-5)
    cache = CacheManager([m.memory_request()], 64 * 12, 3, 512, dtype, DEV)
    cache.allocate_slot()
    s = cache.allocate_slot()
    cache.reserve(s, n)
    cache.flush()
    got = m.forward(x[:n].to(DEV), batch_for("start", [s], [0], [n], cache.scratch_slot), cache.view(0), {})
    torch.testing.assert_close(got.cpu().double(), want[:n], **tol(dtype, 3.0))
    cache.commit(s, n)
    for t in range(n, n + extra):          # the loud tokens leave the window one by one while these run
        cache.reserve(s, t + 1)
        cache.flush()
        got = m.forward(x[t:t + 1].to(DEV), batch_for("extend", [s], [t], [1], cache.scratch_slot), cache.view(0), {})
        torch.testing.assert_close(got.cpu().double(), want[t:t + 1], **tol(dtype, 3.0), msg=lambda e: f"token {t}: {e}")
        cache.commit(s, t + 1)


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("c", LATENT[:3])
def test_latent_attention_in_pieces_and_beside_others(dtype, c):
    """Two sequences fed in pieces of unequal sizes (down to two tokens, across page and ring borders), in one step
    each time, against each alone."""
    from toyinfer_b200.cache import CacheManager
    m, w, mcfg = make_latent(dtype, c, seed=9, edit=sinks_that_matter)
    lens = [203, 131]
    xs = [loud_inputs(n, 56, 20 + i, [5, 63, 64, 100]).to(dtype) for i, n in enumerate(lens)]
    wants = [plain.latent_attention(x.double(), w, "a.", mcfg, 1e-5) for x in xs]
    cache = CacheManager([m.memory_request()], 64 * 16, 4, 512, dtype, DEV)
    slots = [cache.allocate_slot(), cache.allocate_slot()]
    pieces = [[2, 61, 3, 70, 1, 64, 2], [64, 2, 1, 1, 63]]
    fed = [0, 0]
    step = 0
    while any(f < n for f, n in zip(fed, lens)):
        who, news, starts = [], [], []
        for i in range(2):
            if fed[i] < lens[i] and step < len(pieces[i]):
                who.append(i); starts.append(fed[i]); news.append(min(pieces[i][step], lens[i] - fed[i]))
            elif fed[i] < lens[i]:
                who.append(i); starts.append(fed[i]); news.append(lens[i] - fed[i])
        for i, st, nw in zip(who, starts, news):
            cache.reserve(slots[i], st + nw)
        cache.flush()
        mode = "start" if all(st == 0 for st in starts) else "extend" if all(nw == 1 for nw in news) else "mixed"
        x = torch.cat([xs[i][st:st + nw] for i, st, nw in zip(who, starts, news)]).to(DEV)
        got = m.forward(x, batch_for(mode, [slots[i] for i in who], starts, news, cache.scratch_slot), cache.view(0), {}).cpu().double()
        o = 0
        for i, st, nw in zip(who, starts, news):
            torch.testing.assert_close(got[o:o + nw], wants[i][st:st + nw], **tol(dtype, 3.0), msg=lambda e: f"seq {i} at {st}+{nw}: {e}")
            o += nw
            cache.commit(slots[i], st + nw)
            fed[i] = st + nw
        step += 1


# ---------------------------------------------------------------------------
LIGHT = [dict(heads=3, dim=16, vdim=24, decay=[0.9, 0.5, 1.0]), dict(heads=1, dim=40, vdim=150, decay=[0.999]),
         dict(heads=2, dim=128, vdim=8, decay=[0.0, 0.97])]


def make_lightning(dtype, c, hidden=48, seed=4):
    from toyinfer_b200.parts import PartSpec, build_part
    m = build_part("mixer", PartSpec("lightning", {"n_heads": c["heads"], "dim": c["dim"], "vdim": c["vdim"], "decay": c["decay"],
                                                   "eps": 1e-5}), ctx_for(dtype, hidden), "a.")
    return m, bind_random(m, seed, dtype)


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("c", LIGHT)
def test_lightning_scan_chunks_and_single_tokens_agree_with_the_recurrence(dtype, c):
    """A long run of tokens (the chunked form), a short one (the scan), pieces, and 80 single tokens after each
    other, for two sequences of unequal length in one step; a loud early token must still be felt at the end
    where the decay is near one."""
    from toyinfer_b200.cache import CacheManager
    m, w = make_lightning(dtype, c)
    lens = [331, 77]
    xs = []
    for i, n in enumerate(lens):
        x = torch.randn(n + 80, 48, generator=torch.Generator().manual_seed(50 + i))
        x[2] *= 8.0
        xs.append(x.to(dtype))
    wants = [plain.lightning(x.double(), w, "a.", c, 1e-5) for x in xs]
    cache = CacheManager([m.memory_request()], 64 * 16, 4, 1024, dtype, DEV)
    cache.allocate_slot()
    slots = [cache.allocate_slot(), cache.allocate_slot()]
    t = tol(dtype, 2.0)
    x = torch.cat([xs[0][:lens[0]], xs[1][:lens[1]]]).to(DEV)
    got = m.forward(x, batch_for("start", slots, [0, 0], lens, cache.scratch_slot), cache.view(0), {}).cpu().double()
    torch.testing.assert_close(got[:lens[0]], wants[0][:lens[0]], **t)
    torch.testing.assert_close(got[lens[0]:], wants[1][:lens[1]], **t)
    for k in range(80):
        x = torch.stack([xs[0][lens[0] + k], xs[1][lens[1] + k]]).to(DEV)
        got = m.forward(x, batch_for("extend", slots, [lens[0] + k, lens[1] + k], [1, 1], cache.scratch_slot), cache.view(0), {}).cpu().double()
        torch.testing.assert_close(got[0], wants[0][lens[0] + k], **t, msg=lambda e: f"token {k}: {e}")
        torch.testing.assert_close(got[1], wants[1][lens[1] + k], **t, msg=lambda e: f"token {k}: {e}")
    # a slot that is given back and handed out again starts from zero; pieces give what the whole gave
    state_after = cache.view(0).state[slots[0]].clone()
    cache.release(slots[0])
    s = cache.allocate_slot()
    assert s == slots[0] and float(cache.view(0).state[s].abs().max()) == 0.0
    fed = 0
    for piece in [2, 190, 1, 64, 200, 500]:
        piece = min(piece, lens[0] + 80 - fed)
        if piece <= 0:
            break
        mode = "start" if fed == 0 else "extend" if piece == 1 else "mixed"
        got = m.forward(xs[0][fed:fed + piece].to(DEV), batch_for(mode, [s], [fed], [piece], cache.scratch_slot), cache.view(0), {}).cpu().double()
        torch.testing.assert_close(got, wants[0][fed:fed + piece], **t, msg=lambda e: f"piece at {fed}: {e}")
        fed += piece
    torch.testing.assert_close(cache.view(0).state[s], state_after, rtol=2e-3, atol=2e-3)


# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DT)
def test_squared_relu_feed_forward(dtype):
    from toyinfer_b200.parts import PartSpec, build_part
    f = build_part("feed_forward", PartSpec("relu2", {"intermediate_size": 100}), ctx_for(dtype, 40), "m.")
    w = bind_random(f, 2, dtype)
    x = (3 * torch.randn(11, 40, generator=torch.Generator().manual_seed(3))).to(dtype)
    torch.testing.assert_close(f.forward(x.to(DEV), None).cpu().double(), plain.dense_ff(x.double(), w, "m."), **tol(dtype))


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("experts,top,M", [(5, 2, 70), (3, 1, 1), (4, 4, 9), (40, 3, 200), (2, 2, 130), (3, 1, 400)])
@pytest.mark.parametrize("hidden,ff", [(40, 36), (136, 200)])
def test_table_routed_experts(dtype, experts, top, M, hidden, ff):
    """(Rows of 40 and 36 elements run on the CUDA cores in both types; 136 and 200 on the tensor cores in bfloat16.)"""
    from toyinfer_b200.parts import PartSpec, build_part
    vocab, limit = 23, 0.7
    f = build_part("feed_forward", PartSpec("table_moe", {"n_experts": experts, "top": top, "intermediate_size": ff, "limit": limit,
                                                          "vocab_size": vocab}), ctx_for(dtype, hidden), "m.")
    w = bind_random(f, 5, dtype)
    g = torch.Generator().manual_seed(6)
    x = (4 * torch.randn(M, hidden, generator=g)).to(dtype)          # large enough for both clamps to act
    ids = torch.randint(0, vocab, (M,), generator=g).tolist()
    got = f.forward(x.to(DEV), batch_for("start", [0], [0], [M], 1, ids=[ids])).cpu().double()
    cfg = {"router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    want = plain.table_moe(x.double(), ids, w, "m.", cfg)
    gate = x.double() @ w["m.e0.gate"].double().T
    assert (gate > limit).any() and (gate < -limit).any()
    torch.testing.assert_close(got, want, **tol(dtype, 2.0))
