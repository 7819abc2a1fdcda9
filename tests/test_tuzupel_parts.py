"""The mechanisms of the Tuzupel decoder one by one, each kernel against the formula written out in float64: the residual
in lanes, the gated linear recurrence row by row and in chunks, over steps and shuffled slots, the router with softmax
scores, a choice bias and a constant, the clamped gated activation, the sum over routed, identity and shared experts, and
attention whose queries stay in their block of positions or in a window, with one key made to stand out at every edge."""
import math

import pytest
import torch

from tuzupel_helpers import attn, config, lat, layer, lively_tensors, plain, plain_logits, rel_err, write_model

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from beglin_b200.csrc import ops as o
    return o


@pytest.mark.parametrize("n,d,T", [(1, 40, 5), (2, 256, 33), (3, 75, 1), (4, 1031, 7), (8, 64, 3)])
@pytest.mark.parametrize("owed", ["none", "float", "bfloat16", "parts"])
def test_lanes_write_read_norm(n, d, T, owed):
    g = torch.Generator().manual_seed(n * 1000 + d)
    lanes = torch.randn(n, T, d, generator=g)
    mix, outw, inw = torch.randn(n, n, generator=g), torch.randn(n, generator=g), torch.randn(n, generator=g)
    w = 1.0 + 0.3 * torch.randn(d, generator=g)
    y = None
    if owed == "float":
        y = torch.randn(T, d, generator=g)
    elif owed == "bfloat16":
        y = torch.randn(T, d, generator=g).to(torch.bfloat16)
    elif owed == "parts":
        y = torch.randn(3, T, d, generator=g)
    L = lanes.double()
    if y is not None:
        yy = y.double().reshape(-1, T, d).sum(0)
        L = torch.einsum("ab,atd->btd", mix.double(), L) + outw.double()[:, None, None] * yy
    z = torch.einsum("a,atd->td", inw.double(), L)
    want_h = plain.rms_unit(z, 1e-5) * w.double()
    dl = lanes.to(DEV).contiguous()
    h = torch.empty(T, d, device=DEV)
    zz = torch.empty(T, d, device=DEV)
    kw = {} if y is None else {"owed": y.to(DEV), "mix": mix.to(DEV), "out_weights": outw.to(DEV)}
    ops().lane_step(dl, in_weights=inw.to(DEV), norm_weight=w.to(DEV), eps=1e-5, h=h, z=zz, **kw)
    assert rel_err(h, want_h) < 2e-6 and rel_err(zz, z) < 2e-6 and rel_err(dl, L) < 2e-6
    # the sum of the lanes at some rows only, with something owed: nothing is written back
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
    before = lanes.to(DEV).contiguous()
    s = torch.empty(2, d, device=DEV)
    ops().lane_step(before, z=s, rows=rows, **kw)
    assert torch.equal(before.cpu(), lanes)
    assert rel_err(s, L.sum(0)[[T - 1, 0]]) < 2e-6
    hb = torch.empty(T, d, device=DEV, dtype=torch.bfloat16)
    ops().lane_step(before, in_weights=inw.to(DEV), norm_weight=w.to(DEV), eps=1e-5, h=hb, **kw)
    assert rel_err(hb, want_h) < 1e-2


def recurrence(gr, gi, u, y, br, bi, lam, S, scale=8.0):
    """float64, token by token: gr, gi, u, y [T, W]; returns (out [T, W], final state)."""
    out = torch.zeros_like(u)
    sp = scale * torch.nn.functional.softplus(lam)
    for t in range(u.shape[0]):
        r, i = torch.sigmoid(gr[t] + br), torch.sigmoid(gi[t] + bi)
        a = torch.exp(-r * sp)
        S = a * S + torch.sqrt(1.0 - a * a) * (i * u[t])
        out[t] = S * plain.gelu_tanh(y[t])
    return out, S


@pytest.mark.parametrize("W,blocks", [(1, 1), (6, 3), (130, 2), (256, 1), (75, 5)])
def test_recurrence_row_by_row_in_chunks_over_steps_and_slots(W, blocks):
    """Three steps over four requests in shuffled slots with NaN in everything unwritten: portions of 1 to 200 rows, the
    long ones in chunks, against the recurrence token by token; decays from a few tokens to thousands."""
    o = ops()
    g = torch.Generator().manual_seed(W)
    bs = W // blocks
    lam = (-9.0 * torch.rand(W, generator=g)).double()
    br, bi = torch.randn(W, generator=g).double(), torch.randn(W, generator=g).double()
    decay = torch.empty(W, device=DEV)
    o.rglru_softplus(lam.float().to(DEV), 8.0, decay)
    assert rel_err(decay, 8.0 * torch.nn.functional.softplus(lam)) < 1e-6
    slots_total, size = 6, W + 5
    state = torch.full((slots_total, size), float("nan"), device=DEV)
    slot_of = [4, 0, 5, 2]
    state[slot_of, :W] = 0.0
    S = [torch.zeros(W, dtype=torch.float64) for _ in range(4)]
    from beglin_b200.engine.batch import cut_long_requests
    for lens in ([200, 1, 64, 3], [1, 70, 1, 129], [63, 2, 1, 1]):
        T = sum(lens)
        gr, gi, u, y = (torch.randn(T, W, generator=g).double() for _ in range(4))
        gates = torch.empty(blocks, T, 2 * bs)
        for b in range(blocks):
            gates[b, :, :bs] = gr[:, b * bs:(b + 1) * bs]
            gates[b, :, bs:] = gi[:, b * bs:(b + 1) * bs]
        src = torch.full((T, W + 3), float("nan"))
        src[:, 3:] = y
        starts = [sum(lens[:i]) for i in range(4)]
        want = torch.zeros(T, W, dtype=torch.float64)
        for i in range(4):
            sl = slice(starts[i], starts[i] + lens[i])
            want[sl], S[i] = recurrence(gr[sl], gi[sl], u[sl], y[sl], br, bi, lam, S[i])
        short, chunks, longs = cut_long_requests(starts, lens, 32, 64)
        dev = lambda a: torch.from_numpy(a).to(DEV)
        out = torch.full((T, W), float("nan"), device=DEV)
        args = (gates.to(DEV), u.float().to(DEV), src.to(DEV), 3, br.float().to(DEV), bi.float().to(DEV), decay, state,
                torch.tensor(slot_of, dtype=torch.int32, device=DEV))
        if short.shape[0]:
            o.rglru_scan(*args, dev(short), short.shape[0], out)
        o.rglru_scan(*args, None, 0, out, chunked=(dev(chunks), chunks.shape[0], dev(longs), longs.shape[0], 32))
        assert rel_err(out, want) < 5e-6
        for i in range(4):
            assert rel_err(state[slot_of[i], :W], S[i]) < 5e-6
    assert torch.isnan(state[[1, 3]]).all() and torch.isnan(state[:, W:]).all()


def test_recurrence_keeps_a_far_token():
    """One token 900 rows back whose input gate is open while all others are shut: a decay of e^(-8 r softplus(lam)) per
    row with lam = -12 keeps it, lam = -4 fades it."""
    o = ops()
    T, W = 901, 2
    gr = torch.zeros(T, W)
    gi = torch.full((T, W), -40.0)
    gi[0] = 40.0
    u, y = torch.ones(T, W), torch.ones(T, W)
    lam = torch.tensor([-12.0, -4.0])
    decay = torch.empty(W, device=DEV)
    o.rglru_softplus(lam.to(DEV), 8.0, decay)
    gates = torch.cat([gr, gi], dim=1).view(1, T, 2 * W).contiguous()
    state = torch.zeros(1, W, device=DEV)
    out = torch.empty(T, W, device=DEV)
    reqs = torch.tensor([[0, 0, T]], dtype=torch.int32, device=DEV)
    zero = torch.zeros(W, device=DEV)
    o.rglru_scan(gates.to(DEV), u.to(DEV), y.to(DEV), 0, zero, zero, decay, state, torch.zeros(1, dtype=torch.int32, device=DEV), reqs, 1, out)
    want, _ = recurrence(gr.double(), gi.double(), u.double(), y.double(), torch.zeros(W).double(), torch.zeros(W).double(),
                         lam.double(), torch.zeros(W).double())
    assert rel_err(out[-1], want[-1]) < 1e-4          # (900 products of decays, each rounded)
    assert float(out[-1, 0]) > 0.05 * float(out[0, 0]) and float(out[-1, 1]) < 1e-6 * float(out[0, 1])


@pytest.mark.parametrize("T,d,E,top", [(1, 8, 2, 1), (7, 24, 5, 2), (300, 64, 20, 4), (19, 33, 9, 9)])
@pytest.mark.parametrize("mode", ["softmax", "sigmoid", "none"])
def test_router_scores_choice_bias_and_constant(T, d, E, top, mode):
    o = ops()
    g = torch.Generator().manual_seed(T + E)
    h = torch.randn(T, d, generator=g)
    W = torch.randn(E, d, generator=g) / math.sqrt(d)
    bias = 0.2 * torch.randn(E, generator=g)
    z = h.double() @ W.double().T
    s = {"softmax": torch.softmax(z, -1), "sigmoid": torch.sigmoid(z), "none": z}[mode]
    choice = s + bias.double()
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    w = torch.empty(T, top, device=DEV)
    o.route(h.to(DEV), W.to(DEV), top, ids, w, sigmoid=mode, bias=bias.to(DEV), scale=2.5)
    for t in range(T):
        order = sorted(range(E), key=lambda e: (-float(choice[t, e]), e))[:top]
        assert ids[t].tolist() == order, t
        assert rel_err(w[t], 2.5 * s[t, order]) < 2e-5
    # equal scores: the lower index first
    if E >= 2:
        ids2 = torch.empty(1, 2, dtype=torch.int32, device=DEV)
        w2 = torch.empty(1, 2, device=DEV)
        o.route(torch.zeros(1, d, device=DEV), W.to(DEV), 2, ids2, w2, sigmoid=mode)
        assert ids2[0].tolist() == [0, 1]


def test_clamped_gate_and_the_sum_over_routed_identity_and_shared_experts():
    o = ops()
    g = torch.Generator().manual_seed(5)
    T, d, top, n_real, A = 9, 40, 3, 4, 27
    gu = 4.0 * torch.randn(A, 2 * 11 + 8, generator=g)
    act = torch.empty(A, 11, device=DEV)
    o.glu_clamped(gu.to(DEV), act, 1.5)
    gg, uu = gu[:, :11].double().clamp(max=1.5), gu[:, 11:22].double().clamp(-1.5, 1.5)
    assert rel_err(act, gg * torch.sigmoid(1.702 * gg) * (uu + 1.0)) < 2e-6
    assert float(gu[:, :11].min()) < -1.5 and float(gu.max()) > 1.5           # the gate is clamped above only
    yp = torch.randn(A, d, generator=g)
    ids = torch.randint(0, n_real + 2, (T, top), generator=g).to(torch.int32)
    row_of = torch.randperm(A, generator=g).to(torch.int32)
    w = torch.rand(A, generator=g)
    h = torch.randn(T, d, generator=g)
    shared, sg = torch.randn(T, d, generator=g), torch.randn(T, 3, generator=g)
    want = torch.zeros(T, d, dtype=torch.float64)
    for t in range(T):
        for j in range(top):
            a = t * top + j
            want[t] += w[a].double() * (yp[row_of[a]].double() if ids[t, j] < n_real else h[t].double())
    out = torch.empty(T, d, device=DEV)
    o.route_combine_ext(yp.to(DEV), w.to(DEV), row_of.to(DEV), ids.view(-1).to(DEV), n_real, h.to(DEV), out, top)
    assert rel_err(out, want) < 2e-6
    o.route_combine_ext(yp.to(DEV), w.to(DEV), row_of.to(DEV), ids.view(-1).to(DEV), n_real, h.to(DEV), out, top,
                        shared=shared.to(DEV), sg=sg.to(DEV)[:, 1])
    assert rel_err(out, want + torch.sigmoid(sg[:, 1].double())[:, None] * shared.double()) < 2e-6


def banded_reference(base, dims, factor, low, high, original):
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        wl = 2.0 * math.pi / f
        if wl < original / high:
            out.append(f)
        elif wl > original / low:
            out.append(f / factor)
        else:
            t = (original / wl - low) / (high - low)
            out.append((1 - t) * f / factor + t * f)
    return out


def test_band_scaled_frequencies_have_all_three_bands():
    from beglin_b200.models.tuzupel import BandScaling, banded_frequencies
    got = banded_frequencies(1000.0, 24, BandScaling(factor=4.0, low=0.5, high=8.0, original=128.0))
    want = banded_reference(1000.0, 24, 4.0, 0.5, 8.0, 128.0)
    plain_f = [1000.0 ** (-2.0 * i / 24) for i in range(12)]
    assert got == pytest.approx(want, rel=1e-14) and got == pytest.approx(plain.banded_frequencies(
        1000.0, 24, {"factor": 4.0, "low": 0.5, "high": 8.0, "original": 128.0}), rel=1e-14)
    kinds = {"kept" if a == b else "divided" if abs(a - b / 4.0) < 1e-15 else "blended" for a, b in zip(got, plain_f)}
    assert kinds == {"kept", "divided", "blended"}


# ---------------------------------------------------------------------------------------------- one key that stands out
def standout(mixer):
    """A model of ONE layer without a feed-forward in which token id 1 lives on feature 0 of the residual, which no other
    token touches, and every token has the same positive feature 1."""
    d, vocab = 32, 12
    cfg = config(vocab, d, 1e-6, [layer(mixer)])
    t = lively_tensors(cfg, 1, torch.float32)
    t["embed"] = torch.randn(vocab, d, generator=torch.Generator().manual_seed(3)) * 0.3
    t["embed"][1] = 0.0
    t["embed"][:, 0] = 0.0
    t["embed"][1, 0] = 3.0
    t["embed"][:, 1] = 2.0
    t["l0.norm1"] = torch.zeros(d)
    return cfg, t


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["block", "window"])
def test_a_key_that_stands_out_at_every_edge(tmp_path, dtype, kind):
    """Every query points along the key of token 1, in a feature that does not turn, under a scale that lets such a key
    carry the softmax wherever it is seen.  Queries that see a token 1 just inside their block of positions or window and
    queries that see it just outside, in prompts and in single tokens, over pages of 16: the logits are those of the plain
    implementation, and the plain implementation itself says that an edge one position off gives other logits."""
    size = 37
    small = lambda shape, seed: torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * 0.02
    m = "l0.mix."
    if kind == "block":
        cfg, t = standout(attn(2, 1, 64, 64, 0.25, block=size, rot=16, base=100.0))
        t[m + "q"], t[m + "k"] = small(t[m + "q"].shape, 7), small(t[m + "k"].shape, 8)
        t[m + "k"][40] = 0.0
        t[m + "k"][40, 0] = 2.0                          # a key's feature 40 is the input's feature 0: token 1 alone
        t[m + "q"][[40, 64 + 40]] = 0.0
        t[m + "q"][[40, 64 + 40], 1] = 1.0               # a query's feature 40 is the input's feature 1: every token
        t[m + "q.norm"], t[m + "k.norm"] = torch.ones(64), torch.ones(64)
    else:
        cfg, t = standout(lat(2, 64, 64, 64, 0.5, window=size))
        t[m + "q"], t[m + "dkv"], t[m + "uk"] = small(t[m + "q"].shape, 7), small(t[m + "dkv"].shape, 8), small(t[m + "uk"].shape, 9)
        t[m + "dkv"][40] = 0.0
        t[m + "dkv"][40, 0] = 2.0
        t[m + "uk"][[40, 64 + 40]] = 0.0
        t[m + "uk"][[40, 64 + 40], 40] = 1.0
        t[m + "q"][[40, 64 + 40]] = 0.0
        t[m + "q"][[40, 64 + 40], 1] = 1.0
        t[m + "dkv.norm"] = torch.ones(64)
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = write_model(str(tmp_path / "m"), cfg, {k: v.to(stored) for k, v in t.items()})
    # token 1 at the edges of the blocks [0, 37), [37, 74), [74, 111); for windows (whose keys carry no position, so that
    # two tokens 1 in a window are one value) far apart: the queries at 41 and 116 are the last that see them
    ids = [2 + (i * 7) % 10 for i in range(130)]
    for p in ((5, 36, 37, 73, 74, 100) if kind == "block" else (5, 80)):
        ids[p] = 1
    want = plain_logits(folder, ids)
    from beglin_b200 import Engine
    import replay_lib as rl
    tol = 3e-5 if dtype == "float32" else 4e-2
    for way in ("whole", "cut"):
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=192, page_size=16, max_requests=2, kv_split=64)
        if way == "whole":
            steps = [{"entries": [{"id": "a", "tokens": ids, "want": list(range(130))}], "end": ["a"]}]
        else:
            steps = [{"entries": [{"id": "a", "tokens": ids[:35], "want": list(range(35))}]},
                     {"entries": [{"id": "a", "tokens": ids[35:72], "want": list(range(37))}]}]
            steps += [{"entries": [{"id": "a", "tokens": [ids[i]], "want": [0]}], "end": ["a"] if i == 129 else []}
                      for i in range(72, 130)]
        got = rl.run_in_process(eng, steps)
        rows = torch.stack([got[("a", p)] for p in range(130)])
        assert rel_err(rows, want) < tol, way
    # the same weights under an edge one position off: other logits where the edge passes a token 1
    cfg_w, w = plain.read_folder(folder, torch.float64)
    for other in (size - 1, size + 1):
        cfg_w["layers"][0]["mixer"]["mask"]["size"] = other
        moved = plain.forward(cfg_w, w, ids)
        assert rel_err(moved, want) > 0.3, other
