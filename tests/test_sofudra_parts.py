"""Each mechanism of the Sofudra decoder alone, kernel against the plain implementation's function (or a closed form
written here): the decayed state token by token and in chunks, attention with learned sinks, squashed scores, windows
and values of another size on CUDA cores and on tensor cores, per-head norms with stretched rotation and cache append,
the gate per head, the norm with a sigmoid gate behind it, the sum of scaled branches with two norms, and the tanh
form of GELU."""
import math

import pytest
import torch

from sofudra_helpers import plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def ops():
    from beglin_b200.csrc import ops as o
    return o


def close(got, want, tol):
    got, want = got.double().cpu(), want.double().cpu()
    assert torch.isfinite(got).all()
    err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
    assert err < tol, err


# ----------------------------------------------------------------------------- the decayed state
def plain_decayed(q, k, v, decay, S):
    """q, k [T, H, n], v [T, H, nv] (after their activations), S [H, n, nv] advanced in place -> o [T, H, nv]."""
    T, H, _ = q.shape
    o = torch.zeros(T, H, v.shape[2], dtype=torch.float64)
    for t in range(T):
        for a in range(H):
            S[a] = decay[a] * S[a] + torch.outer(k[t, a], v[t, a])
            o[t, a] = S[a].T @ q[t, a]
    return o


def run_decayed(src, H, n, nv, decay, state, slots, lens, chunked):
    """One step over requests of `lens` rows; `src` [T, q | k | v | extra] or partial sums of it."""
    from beglin_b200.engine.batch import cut_long_requests
    o = ops()
    T = src.shape[-2]
    starts = [sum(lens[:i]) for i in range(len(lens))]
    y = torch.full((T, H * nv), float("nan"), dtype=torch.float32, device=DEV)
    chunk = o.decay_attention_chunk(n, nv)
    dev = lambda a: torch.from_numpy(a).to(DEV)
    if chunked:
        if chunk == 0:
            pytest.skip("heads of this size run token by token only")
        short, blocks, longs = cut_long_requests(starts, lens, chunk, 16)
        o.decay_attention(src, 0, H * n, 2 * H * n, decay, state, slots, dev(short), short.shape[0], y, H, n, nv,
                          dev(blocks), blocks.shape[0], dev(longs), longs.shape[0])
    else:
        reqs = torch.tensor([[i, s, m] for i, (s, m) in enumerate(zip(starts, lens))], dtype=torch.int32, device=DEV)
        o.decay_attention(src, 0, H * n, 2 * H * n, decay, state, slots, reqs, len(lens), y, H, n, nv)
    return y


@pytest.mark.parametrize("H,n,nv", [(1, 1, 1), (3, 6, 10), (2, 14, 5), (4, 32, 32), (2, 64, 64), (1, 128, 128), (2, 33, 7), (1, 96, 40), (1, 300, 40),
                                    (2, 200, 3)])
@pytest.mark.parametrize("chunked", [False, True])
@pytest.mark.parametrize("parts", [1, 3])
def test_decayed_state(H, n, nv, chunked, parts):
    """Three steps over four requests of unequal lengths (one and two tokens, a few, several chunks and a ragged last
    one) whose states lie in shuffled slots of a slab that held NaN before the first step wrote zeros; decays of 0, 1 and
    between.  Outputs and the states behind every step against the recurrence written out token by token."""
    g = torch.Generator().manual_seed(H * n + nv)
    decay = ([0.0, 1.0, 0.93, 0.5] * 2)[:H] if H > 1 else [0.97]
    W = 2 * H * n + H * nv + 3
    slots = torch.tensor([5, 0, 3, 2], dtype=torch.int32, device=DEV)
    slab = torch.full((7, H * n * nv + 4), float("nan"), dtype=torch.float32, device=DEV)
    slab[slots.long(), :H * n * nv] = 0.0
    S = [torch.zeros(H, n, nv, dtype=torch.float64) for _ in range(4)]
    dec = torch.tensor(decay, dtype=torch.float32, device=DEV)
    for lens in ([1, 150, 17, 2], [70, 1, 64, 16], [15, 129, 1, 200]):
        T = sum(lens)
        src = torch.randn(parts, T, W, generator=g) if parts > 1 else torch.randn(T, W, generator=g)
        rows = (src.double().sum(0) if parts > 1 else src.double())
        act = plain.silu(rows)
        q, k = act[:, :H * n].reshape(T, H, n), act[:, H * n:2 * H * n].reshape(T, H, n)
        v = act[:, 2 * H * n:2 * H * n + H * nv].reshape(T, H, nv)
        want, r0 = [], 0
        for i, m in enumerate(lens):
            want.append(plain_decayed(q[r0:r0 + m], k[r0:r0 + m], v[r0:r0 + m], decay, S[i]))
            r0 += m
        y = run_decayed(src.to(DEV), H, n, nv, dec, slab, slots, lens, chunked)
        tol = 1e-5 if n > 1 else 3e-5              # (a single feature: nothing averages the rounding of its products)
        close(y.reshape(T, H, nv), torch.cat(want), tol)
        for i in range(4):
            close(slab[int(slots[i]), :H * n * nv].reshape(H, n, nv), S[i], tol)
    assert torch.isnan(slab[[1, 4, 6]]).all() and torch.isnan(slab[:, H * n * nv:]).all()     # nothing else was written


def test_decayed_state_keeps_a_far_token():
    """One token, 700 back, whose key is the only one aligned with the last query, its value scaled up: with a decay of 1
    its value is what the last row returns; with 0.99 it has faded by 0.99^700."""
    H, n, nv, T = 2, 16, 8, 701
    g = torch.Generator().manual_seed(3)
    q = torch.rand(T, H, n, generator=g, dtype=torch.float64) * 0.01
    k = torch.rand(T, H, n, generator=g, dtype=torch.float64) * 0.01
    v = torch.rand(T, H, nv, generator=g, dtype=torch.float64)
    k[0], q[T - 1], v[0] = 3.0, 3.0, 50.0
    # the kernel applies silu to what it reads: feed it the inverse on positive values (found by bisection)
    def inv_silu(y):
        lo, hi = torch.zeros_like(y), torch.full_like(y, 100.0)
        for _ in range(80):
            mid = (lo + hi) / 2
            big = plain.silu(mid) > y
            hi, lo = torch.where(big, mid, hi), torch.where(big, lo, mid)
        return lo
    src = torch.cat([inv_silu(q.reshape(T, -1)), inv_silu(k.reshape(T, -1)), inv_silu(v.reshape(T, -1))], dim=1).float()
    act = plain.silu(src.double())
    q2, k2 = act[:, :H * n].reshape(T, H, n), act[:, H * n:2 * H * n].reshape(T, H, n)
    v2 = act[:, 2 * H * n:].reshape(T, H, nv)
    decay = [1.0, 0.99]
    for chunked in (False, True):
        slab = torch.zeros(1, H * n * nv, dtype=torch.float32, device=DEV)
        y = run_decayed(src.to(DEV), H, n, nv, torch.tensor(decay, device=DEV), slab, torch.zeros(1, dtype=torch.int32, device=DEV),
                        [T], chunked)
        want = plain_decayed(q2, k2, v2, decay, torch.zeros(H, n, nv, dtype=torch.float64))
        close(y.reshape(T, H, nv), want, 2e-5)
        last = y.reshape(T, H, nv)[T - 1].cpu()
        assert float(last[0].min()) > 0.9 * 9.0 * n * 50.0 and float(last[1].max()) < 0.01 * 9.0 * n * 50.0


# ----------------------------------------------------------------------------- attention
def scattered_tables(lengths, page, n_pages, seed):
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(n_pages, generator=g).tolist()
    width = max(-(-n // page) for n in lengths)
    table = torch.full((len(lengths), width), -1, dtype=torch.int32)
    for r, n in enumerate(lengths):
        for i in range(-(-n // page)):
            table[r, i] = order.pop()
    return table


def run_attention(q, keys, vals, lengths, new, scale, window, sink, cap, dtype, page=16, split=64, prefer="auto", decode=False):
    """Requests with `lengths[r]` cached positions of which the last `new[r]` are the step's rows; q[r] holds the
    queries of those rows.  Returns (rows [T, H, vd], the kernel that ran)."""
    o = ops()
    H, hd = q[0].shape[1:]
    G, vd = keys[0].shape[1], vals[0].shape[2]
    n_pages = sum(-(-n // page) for n in lengths) + 3
    table = scattered_tables(lengths, page, n_pages, 7)
    pool = torch.full((n_pages, G * page * (hd + vd)), float("nan"), dtype=dtype)
    for r, n in enumerate(lengths):
        for p in range(n):
            pg = pool[int(table[r, p // page])]
            pg[:G * page * hd].view(G, page, hd)[:, p % page] = keys[r][p].to(dtype)
            pg[G * page * hd:].view(G, page, vd)[:, p % page] = vals[r][p].to(dtype)
    if hd == vd:
        pool = pool.view(n_pages, 2, G, page, hd)
    rows = torch.cat(q).to(dtype)
    T = rows.shape[0]
    positions = torch.cat([torch.arange(n - m, n) for n, m in zip(lengths, new)]).int()
    kernel, bq, tile = o.attention_plan(H // G, hd, dtype, decode, prefer, page, vd=vd, softcap=bool(cap), learned_sink=sink is not None)
    blocks, r0 = [], 0
    for r, m in enumerate(new):
        blocks += [[r, r0 + f, min(bq, m - f)] for f in range(0, m, bq)]
        r0 += m
    qblk = torch.tensor(blocks, dtype=torch.int32, device=DEV)
    out = torch.empty(T, H * vd, dtype=dtype, device=DEV)
    o.attention(rows.reshape(T, H * hd).to(DEV), H * hd, pool.to(DEV), table.to(DEV), positions.to(DEV), qblk, len(blocks),
                int(positions.max()), T, H, G, hd, window or 0, split, tile, bq, scale, out, o.new_status(DEV), kernel, vd=vd,
                sink_weight=None if sink is None else sink.float().to(DEV), softcap=cap or 0.0)
    return out.reshape(T, H, vd), kernel


def plain_rows(q, keys, vals, lengths, new, scale, window, sink, cap):
    """The oracle's attention over each whole sequence (queries of the cached positions do not matter: zeros), the rows
    of the step taken out."""
    out = []
    for r, (n, m) in enumerate(zip(lengths, new)):
        full = torch.zeros(n, *q[r].shape[1:], dtype=torch.float64)
        full[n - m:] = q[r]
        out.append(plain.softmax_attention(full, keys[r], vals[r], scale, window=window, sink=sink, cap=cap)[n - m:])
    return torch.cat(out)


@pytest.mark.parametrize("H,G,hd,vd,window,cap", [(3, 1, 10, 6, 13, None), (4, 2, 12, 12, 40, 5.0), (2, 2, 16, 24, None, 1.0),
                                                    (6, 3, 64, 32, 100, 30.0), (2, 1, 128, 128, 70, None), (4, 4, 8, 2, 1, 2.0),
                                                    (8, 1, 64, 64, None, 30.0), (6, 2, 48, 48, 40, None)])
@pytest.mark.parametrize("with_sink", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_with_learned_sink_and_squashed_scores(H, G, hd, vd, window, cap, with_sink, dtype):
    """Three requests of unequal lengths in one step: a prompt's portion, a single decoded token far into its sequence,
    and a short first portion.  Scores large enough for the squashing to matter; sinks above, among and below them."""
    g = torch.Generator().manual_seed(H * hd + vd)
    lengths, new = [150, 333, 9], [37, 1, 9]
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    keys, vals, q = [rnd(n, G, hd) for n in lengths], [rnd(n, G, vd) for n in lengths], [rnd(m, H, hd) for m in new]
    if dtype == torch.bfloat16:
        keys, vals, q = [[t.to(dtype).double() for t in ts] for ts in (keys, vals, q)]
    sink = (torch.tensor([4.0, -20.0, 0.0, 1.5, 8.0, -1.0, 2.5, 0.3], dtype=torch.float64)[:H]) if with_sink else None
    scale = 2.5 / math.sqrt(hd)
    got, _ = run_attention(q, keys, vals, lengths, new, scale, window, sink, cap, dtype)
    want = plain_rows(q, keys, vals, lengths, new, scale, window, sink, cap)
    close(got, want, 5e-6 if dtype == torch.float32 else 1.5e-2)
    if cap is not None and window != 1:            # the squashing matters here
        far = plain_rows(q, keys, vals, lengths, new, scale, window, sink, None)
        assert float((far - want).abs().max() / want.abs().max()) > 1e-2


@pytest.mark.parametrize("H,G,hd,window", [(6, 2, 64, 100), (4, 1, 128, None), (8, 1, 64, None), (2, 2, 128, 70), (2, 2, 128, 1),
                                           (3, 1, 64, 2), (2, 1, 128, 17)])
@pytest.mark.parametrize("how", ["tcgen05", "mma", "decode"])
@pytest.mark.parametrize("cap,with_sink", [(30.0, False), (4.0, False), (None, True), (6.0, True)])
def test_tensor_core_attention(H, G, hd, window, how, cap, with_sink):
    """The tensor-core kernels (tcgen05 for portions, mma.sync for portions and for single tokens over split keys) with
    squashed scores and learned sinks, pages of 16 and of 64, against the oracle; left to itself the plan picks the
    tcgen05 kernel for portions of these sizes."""
    g = torch.Generator().manual_seed(H * hd)
    decode = how == "decode"
    lengths, new = ([150, 333, 9, 600], [1, 1, 1, 1]) if decode else ([150, 333, 9], [37, 130, 9])
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64).to(torch.bfloat16).double()
    keys, vals = [rnd(n, G, hd) for n in lengths], [rnd(n, G, hd) for n in lengths]
    q = [rnd(m, H, hd) for m in new]
    sink = torch.tensor([3.0, -20.0, 0.0, 1.5, 6.0, -1.0, 2.5, 0.3], dtype=torch.float64)[:H] if with_sink else None
    scale = 2.0 / math.sqrt(hd)
    for page in (16, 64):
        got, kernel = run_attention(q, keys, vals, lengths, new, scale, window, sink, cap, torch.bfloat16, page=page, split=256,
                                    prefer="auto" if how == "tcgen05" else "mma", decode=decode)
        assert kernel == {"decode": "mma_keys", "mma": "mma_rows", "tcgen05": "tc_rows"}[how], kernel
        close(got, plain_rows(q, keys, vals, lengths, new, scale, window, sink, cap), 1.5e-2)


@pytest.mark.parametrize("place", ["far", "window_last", "window_out", "page_border", "first"])
@pytest.mark.parametrize("cap", [None, 12.0])
def test_attention_one_key_stands_out(place, cap):
    """Among 600 keys one is made to stand out for the last query: far back, the oldest key of the window, just outside
    it, the last key of a page, or the very first one.  Its value, scaled up, is what the row returns when it is seen,
    and is absent when it is not; a sink as large as that key's score takes half."""
    g = torch.Generator().manual_seed(5)
    L, G, H, hd, vd = 600, 1, 2, 16, 8
    window = {"far": None, "window_last": 100, "window_out": 100, "page_border": None, "first": None}[place]
    at = {"far": 11, "window_last": L - 100, "window_out": L - 101, "page_border": 16 * 20 - 1, "first": 0}[place]
    keys = torch.randn(L, G, hd, generator=g, dtype=torch.float64) * 0.3
    vals = torch.randn(L, G, vd, generator=g, dtype=torch.float64)
    q = torch.randn(1, H, hd, generator=g, dtype=torch.float64) * 0.3
    keys[at, 0] = q[0, 0] / q[0, 0].norm() * 8.0
    q[0, 0] *= 8.0 / q[0, 0].norm()                # the score of that key: 64 (squashed: nearly 12)
    vals[at] *= 30.0
    top = 64.0 if cap is None else cap * math.tanh(64.0 / cap)
    sink = torch.tensor([top, -5.0], dtype=torch.float64)
    got, _ = run_attention([q], [keys], [vals], [L], [1], 1.0, window, sink, cap, torch.float32)
    want = plain_rows([q], [keys], [vals], [L], [1], 1.0, window, sink, cap)
    close(got, want, 1e-5)
    if place != "window_out":
        close(got[0, 0], vals[at, 0] * 0.5, 0.05 if cap is None else 0.2)
    else:
        assert float(got[0, 0].abs().max()) < 1.0


# ----------------------------------------------------------------------------- norms of heads, rotation, append
@pytest.mark.parametrize("nh,nkv,hd,vd,rot,scaling,dtype", [
    (3, 1, 10, 6, 6, (2.5, 64, 4.0, 0.5), torch.float32), (4, 2, 12, 12, 12, (6.0, 512, 24.0, 1.0), torch.float32),
    (2, 2, 16, 24, 4, None, torch.float32), (4, 2, 64, 32, 32, (4.0, 256, 16.0, 2.0), torch.bfloat16),
    (6, 2, 48, 48, 48, (6.0, 512, 24.0, 1.0), torch.float32), (8, 8, 8, 2, 8, (1.0, 16, 2.0, 1.0), torch.float32)])
@pytest.mark.parametrize("parts", [1, 3])
def test_head_norms_stretched_rotation_and_append(nh, nkv, hd, vd, rot, scaling, dtype, parts):
    """Every head of q and k normed by itself with one weight vector for all heads, the leading features rotated in
    halves with this package's stretched frequencies and amplitude, k and v appended to scattered pages; against the
    oracle's norm and rotation."""
    from beglin_b200.models.sofudra import StretchConfig, stretched_frequencies
    o = ops()
    g = torch.Generator().manual_seed(nh * hd + vd)
    lengths, page = [13, 5], 8
    T = sum(lengths)
    positions = torch.cat([torch.arange(900, 900 + lengths[0]), torch.arange(0, lengths[1])]).int()
    row_req = torch.cat([torch.zeros(lengths[0]), torch.ones(lengths[1])]).int()
    table = scattered_tables([900 + lengths[0], lengths[1]], page, 120, 1)
    qd, kd, vdd, extra = nh * hd, nkv * hd, nkv * vd, 5
    src = torch.randn(parts, T, qd + kd + vdd + extra, generator=g) if parts > 1 else torch.randn(T, qd + kd + vdd + extra, generator=g).to(dtype)
    wq, wk = 1 + 0.3 * torch.randn(hd, generator=g), 1 + 0.3 * torch.randn(hd, generator=g)
    eps, base = 1e-5, 50.0
    rows = (src.double().sum(0) if parts > 1 else src.double())
    sc = None if scaling is None else dict(zip(("factor", "original", "fast", "slow"), scaling))
    q = plain.head_norm(rows[:, :qd].reshape(T, nh, hd), wq.double(), eps)
    k = plain.head_norm(rows[:, qd:qd + kd].reshape(T, nkv, hd), wk.double(), eps)
    v = rows[:, qd + kd:qd + kd + vdd].reshape(T, nkv, vd)
    q = plain.turn_halves(q, positions.tolist(), base, rot, sc)
    k = plain.turn_halves(k, positions.tolist(), base, rot, sc)
    freqs, amp = stretched_frequencies(base, rot, None if scaling is None else StretchConfig(*scaling))
    cos_sin = torch.empty(T, rot // 2, 2, dtype=torch.float32, device=DEV)
    o.rope_table(positions.to(DEV), torch.tensor(freqs, dtype=torch.float32, device=DEV), cos_sin, amplitude=amp)
    n_pages = 120
    pool = torch.full((n_pages, nkv * page * (hd + vd)), float("nan"), dtype=dtype, device=DEV)
    q_out = torch.empty(T, qd, dtype=dtype, device=DEV)
    o.qk_norm_rope_append(src.to(DEV), q_out, T, nh, nkv, hd, vd, rot, False, wq.to(DEV), wk.to(DEV), eps, cos_sin,
                          positions.to(DEV), row_req.to(DEV), table.to(DEV), pool, page, None, per_head=True)
    tol = 1e-4 if dtype == torch.float32 else 1e-2       # (an angle of 900 turns of a radian in 32 bits is good to 5e-5)
    close(q_out, q.reshape(T, qd), tol)
    pool = pool.cpu().double()
    for t in range(T):
        p = int(positions[t])
        pg = pool[int(table[int(row_req[t]), p // page])]
        close(pg[:nkv * page * hd].reshape(nkv, page, hd)[:, p % page], k[t], tol)
        close(pg[nkv * page * hd:].reshape(nkv, page, vd)[:, p % page], v[t], tol)
    assert int(torch.isnan(pool).sum()) == pool.numel() - T * (kd + vdd)          # nothing else was written


# ----------------------------------------------------------------------------- gates, norms, sums
@pytest.mark.parametrize("parts", [1, 2])
@pytest.mark.parametrize("H,vd", [(3, 6), (1, 1), (8, 64), (5, 1)])
def test_one_gate_per_head(parts, H, vd):
    g = torch.Generator().manual_seed(H + vd)
    T, col0, W = 7, 11, 11 + H + 4
    out = torch.randn(T, H * vd, generator=g)
    src = torch.randn(parts, T, W, generator=g) if parts > 1 else torch.randn(T, W, generator=g)
    gate = (src.sum(0) if parts > 1 else src)[:, col0:col0 + H]
    want = (out.double().reshape(T, H, vd) * torch.sigmoid(gate.double())[:, :, None]).reshape(T, H * vd)
    od = out.to(DEV)
    ops().sigmoid_gate(od, src.to(DEV), col0, H * vd, gate_per=vd)
    close(od, want, 2e-6)


@pytest.mark.parametrize("inner,dtype", [(18, torch.float32), (128, torch.bfloat16), (1, torch.float32), (300, torch.float32)])
def test_norm_with_a_sigmoid_gate_behind_it(inner, dtype):
    g = torch.Generator().manual_seed(inner)
    T, col = 9, 7
    y = torch.randn(T, inner, generator=g) * 3
    src = torch.randn(T, col + inner + 2, generator=g)
    w = (1 + 0.3 * torch.randn(inner, generator=g))
    want = plain.rms_norm(y.double(), w.double(), 1e-5) * torch.sigmoid(src.double()[:, col:col + inner])
    out = torch.empty(T, inner, dtype=dtype, device=DEV)
    ops().gated_group_rmsnorm(y.to(DEV), src.to(DEV), col, w.to(DEV), 1e-5, 1, out, gate_after=True)
    close(out, want, 3e-6 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("d,lowp", [(72, False), (384, True), (5, False), (1000, True)])
@pytest.mark.parametrize("assign", [False, True])
def test_sum_of_scaled_terms_with_two_norms(d, lowp, assign):
    """x (= or +=) a sum of scaled terms of both number types and of partial sums, then two norms of the same rows."""
    g = torch.Generator().manual_seed(d)
    T = 11
    x = torch.randn(T, d, generator=g)
    a, b = torch.randn(T, d, generator=g), torch.randn(3, T, d, generator=g)
    c = torch.randn(T, d, generator=g).to(torch.bfloat16)
    w1, w2 = 1 + 0.3 * torch.randn(d, generator=g), 1 + 0.3 * torch.randn(d, generator=g)
    want = (0.0 if assign else x.double()) + 0.3 * a.double() - 1.7 * b.double().sum(0) + 0.5 * c.double()
    xd = x.to(DEV)
    odt = torch.bfloat16 if lowp else torch.float32
    o1, o2 = torch.empty(T, d, dtype=odt, device=DEV), torch.empty(T, d, dtype=odt, device=DEV)
    ops().add_terms_norm(xd, [(a.to(DEV), 0.3), (b.to(DEV), -1.7), (c.to(DEV), 0.5)], assign=assign, weight1=w1.to(DEV),
                         weight2=w2.to(DEV), eps=1e-5, out1=o1, out2=o2)
    close(xd, want, 2e-6)
    close(o1, plain.rms_norm(want, w1.double(), 1e-5), 1e-2 if lowp else 3e-6)
    close(o2, plain.rms_norm(want, w2.double(), 1e-5), 1e-2 if lowp else 3e-6)
    ops().add_terms_norm(xd, [(a.to(DEV), 1.0)])                 # a sum alone
    close(xd, want + a.double(), 2e-6)


@pytest.mark.parametrize("parts,dtype", [(1, torch.float32), (1, torch.bfloat16), (3, torch.float32)])
def test_gelu_in_its_tanh_form(parts, dtype):
    g = torch.Generator().manual_seed(parts)
    z = (torch.randn(parts, 6, 50, generator=g) * 3 if parts > 1 else (torch.randn(6, 50, generator=g) * 3).to(dtype))
    out = torch.empty(6, 50, dtype=dtype, device=DEV)
    ops().activation(z.to(DEV), out, "gelu_tanh")
    close(out, plain.gelu_tanh(z.double().sum(0) if parts > 1 else z.double()), 2e-6 if dtype == torch.float32 else 1e-2)
