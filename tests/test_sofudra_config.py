"""The Sofudra decoder's configuration reader, its description as parts, the order of its stages, the tensors it asks for
and the cache needs of its layers; the cutting of long requests into chunks; and the plain implementation's small
functions against closed forms.  No GPU."""
import copy
import math

import numpy as np
import pytest
import torch

from sofudra_helpers import EVEN, ODD, SHARP, attn, config, decayed, gated, layer, par, plain

from beglin_b200.config import ConfigError, load_config
from beglin_b200.engine.batch import cut_long_requests
from beglin_b200.models.sofudra import StretchConfig, stretched_frequencies
from beglin_b200.parts.cache_need import CompositeNeed, FixedStateNeed, PagedKVNeed
from beglin_b200.weights import expected_tensors


def test_reads_every_size_and_constant():
    arch, cfg = load_config(copy.deepcopy(ODD))
    assert arch.name == "Sofudra" and (cfg.vocab, cfg.width, cfg.norm_eps) == (211, 72, 1e-6)
    assert (cfg.embed_scale, cfg.residual_mult, cfg.logit_softcap) == (4.0, 0.4, 20.0)
    assert (cfg.loop.start, cfg.loop.stop, cfg.loop.times) == (1, 3, 3)
    p0, a1 = cfg.layers[0].mixer, cfg.layers[1].mixer
    assert (p0.left.heads, p0.left.kv_heads, p0.left.dim, p0.left.vdim, p0.left.scale, p0.left.softcap) == (3, 1, 10, 6, 0.4, 5.0)
    assert (p0.right.heads, p0.right.dim, p0.right.vdim, p0.right.decay) == (3, 6, 10, (0.5, 0.9, 0.99))
    assert (p0.left_scale, p0.right_scale) == (0.7, 1.3) and p0.left.window is None and p0.left.rot_dims == 0
    assert (a1.heads, a1.kv_heads, a1.dim, a1.vdim, a1.window, a1.rot_dims, a1.rot_base) == (4, 2, 12, 12, 13, 8, 100.0)
    assert a1.stretch == StretchConfig(2.5, 64, 4.0, 0.5) and cfg.layers[3].mixer.stretch is None
    assert cfg.layers[2].ff is None and cfg.layers[0].ff == 100
    assert cfg.to_json_dict() == ODD                                   # and back


def test_stages_follow_the_loop():
    arch, cfg = load_config(copy.deepcopy(ODD))
    spec = arch.build_spec(cfg)
    assert [s.layer for s in spec.order] == [0, 1, 2, 1, 2, 1, 2, 3, 4]
    assert [s.enter for s in spec.order] == [None, 0, None, 0, None, 0, None, None, None]
    assert [l.block for l in spec.layers] == ["parallel", "parallel", "parallel_mixer", "parallel", "parallel_mixer"]
    assert len(spec.entries) == 1 and spec.entries[0].names == {"weight": "loop.in"}
    # a loop from the first layer on; no loop at all
    _, sharp = load_config(copy.deepcopy(SHARP))
    s2 = arch.build_spec(sharp)
    assert [s.layer for s in s2.order] == [0, 1, 0, 1, 2] and [s.enter for s in s2.order] == [0, None, 0, None, None]
    _, even = load_config(copy.deepcopy(EVEN))
    s3 = arch.build_spec(even)
    assert [s.layer for s in s3.order] == [0, 1, 2, 3] and not s3.entries and "loop.in" not in expected_tensors(s3)
    # one pass is a pass: the input mix stands in front of it
    once = copy.deepcopy(ODD)
    once["loop"]["times"] = 1
    s4 = arch.build_spec(load_config(once)[1])
    assert [s.enter for s in s4.order] == [None, 0, None, None, None]


def test_spec_carries_the_options():
    arch, cfg = load_config(copy.deepcopy(ODD))
    spec = arch.build_spec(cfg)
    a = spec.layers[1].mixer
    assert a.sink == "learned" and a.gate is None and a.qk_norm == "head" and a.qk_norm_eps == 1e-6 and not a.qkv_bias
    assert (a.head_dim, a.v_head_dim, a.window, a.scale, a.score_cap) == (12, 12, 13, 0.3, None)
    assert a.position.pairing == "split_half" and a.position.rotary_dim == 8 and len(a.position.frequencies) == 4
    assert a.position.amplitude == pytest.approx(0.1 * math.log(2.5) + 1.0)
    assert spec.layers[3].mixer.position.amplitude == 1.0
    p = spec.layers[0].mixer
    left, right = p.branches
    assert p.scales == (0.7, 1.3) and p.labels == ("left", "right")
    assert left.gate == "head" and not left.sink and left.qkv_bias and left.score_cap == 5.0 and left.position.kind == "none"
    assert left.window is None and (right.n_heads, right.dim, right.vdim, right.decay, right.eps) == (3, 6, 10, (0.5, 0.9, 0.99), 1e-6)
    assert spec.layers[0].feed_forward.activation == "gelu_tanh" and spec.layers[0].block_args == {"residual_mult": 0.4}
    assert spec.embed_scale == 4.0 and spec.logit_softcap == 20.0


def test_tensor_names_and_shapes():
    arch, cfg = load_config(copy.deepcopy(ODD))
    t = expected_tensors(arch.build_spec(cfg))
    shape = lambda n: tuple(t[n].shape)
    assert shape("loop.in") == (72, 144) and shape("embed") == (211, 72) and shape("head") == (211, 72) and shape("final.norm") == (72,)
    assert shape("l0.mix.left.q") == (30, 72) and shape("l0.mix.left.q.b") == (30,) and shape("l0.mix.left.k") == (10, 72)
    assert shape("l0.mix.left.v.b") == (6,) and shape("l0.mix.left.g") == (3, 72) and shape("l0.mix.left.o") == (72, 18)
    assert shape("l0.mix.left.q.norm") == (10,) and shape("l0.mix.left.k.norm") == (10,)
    assert shape("l0.mix.right.q") == (18, 72) and shape("l0.mix.right.k") == (18, 72) and shape("l0.mix.right.v") == (30, 72)
    assert shape("l0.mix.right.g") == (30, 72) and shape("l0.mix.right.norm") == (30,) and shape("l0.mix.right.o") == (72, 30)
    assert shape("l1.mix.q") == (48, 72) and shape("l1.mix.k") == (24, 72) and shape("l1.mix.sink") == (4,) and shape("l1.mix.q.norm") == (12,)
    assert "l1.mix.q.b" not in t and "l1.mix.g" not in t and "l0.mix.left.sink" not in t
    assert shape("l0.mlp.up") == (100, 72) and shape("l0.mlp.down") == (72, 100) and "l0.mlp.act" not in t
    assert "l2.norm2" not in t and "l2.norm1" in t and not any(n.startswith("l2.mlp") for n in t)


def test_cache_needs_follow_the_layers():
    from beglin_b200.parts import registry
    arch, cfg = load_config(copy.deepcopy(ODD))
    spec = arch.build_spec(cfg)
    need = lambda l: registry.mixer_class(l.mixer.kind).cache_need(l.mixer)
    n0, n1 = need(spec.layers[0]), need(spec.layers[1])
    assert isinstance(n0, CompositeNeed) and n0.needs == (PagedKVNeed(1, 10, None, 6), FixedStateNeed((3 * 6 * 10,), "float32"))
    assert n1 == PagedKVNeed(2, 12, 13, None)


def test_every_pass_of_the_loop_has_its_own_cache():
    """A stage is a run of a layer: the cache manager places each of the nine runs, not the five layers; a parallel layer's
    run holds pages for its left branch and a state slot for its right one."""
    from beglin_b200.cache import CacheManager
    from beglin_b200.parts import registry
    arch, cfg = load_config(copy.deepcopy(ODD))
    spec = arch.build_spec(cfg)
    needs = [registry.mixer_class(spec.layers[s.layer].mixer.kind).cache_need(spec.layers[s.layer].mixer) for s in spec.order]
    cache = CacheManager(needs, page_size=8, num_pages=4, max_requests=2)
    assert sorted(cache.stage_group) == list(range(9))
    places = [cache.stage_group[i] for i in (1, 3, 5)]                 # the three passes over layer 1
    assert len({p for p in places}) == 3 and all(p[0] == "kv" and p[1] == places[0][1] for p in places)
    several = cache.stage_group[2]
    assert several[0] == "several" and [p[0] for p in several[1]] == ["kv", "state"]
    assert cache.stage_group[2][1][1] != cache.stage_group[4][1][1]    # another pass, another state


@pytest.mark.parametrize("change,what", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 3), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 5), "even"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 14), "at most"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "glu"), "kind"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][0]["mixer"].pop("right"), "right"),
    (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("decay", [0.5, 0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("decay", [0.5, 0.5, 1.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("softcap", 0.0), "softcap"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.__setitem__("layers", []), "empty"),
    (lambda c: c["layers"][1]["mixer"]["mask"].__setitem__("size", 0), "positive"),
    (lambda c: c["loop"].__setitem__("stop", 9), "loop"),
    (lambda c: c["loop"].__setitem__("times", 0), "loop"),
])
def test_bad_configurations_are_refused(change, what):
    c = copy.deepcopy(ODD)
    change(c)
    with pytest.raises(ConfigError) as e:
        load_config(c)
    assert what in str(e.value)


# ----------------------------------------------------------------------------- stretched frequencies
def test_stretched_frequencies_closed_forms():
    # without stretching: the plain powers and amplitude one
    f, amp = stretched_frequencies(100.0, 8, None)
    assert amp == 1.0 and f == pytest.approx([100.0 ** (-2 * i / 8) for i in range(4)])
    # a ramp that lies wholly behind the pairs leaves them alone; one wholly in front divides all of them
    f_hi, amp = stretched_frequencies(100.0, 8, StretchConfig(4.0, 1e9, 1e-3, 1e-4))
    assert f_hi == pytest.approx(f) and amp == pytest.approx(0.1 * math.log(4.0) + 1.0)
    f_lo, _ = stretched_frequencies(100.0, 8, StretchConfig(4.0, 1.0, 1e3, 1e2))
    assert f_lo[1:] == pytest.approx([x / 4.0 for x in f[1:]]) and f_lo[0] == pytest.approx(f[0])   # lo = hi = 0: pair 0 stays
    # the product's and the oracle's agree (two implementations of the same formulas)
    for base, dims, s in [(300000.0, 40, (6.0, 2048, 24.0, 1.5)), (10.0, 6, (3.0, 16, 2.0, 1.0)), (1000.0, 24, (2.5, 64, 4.0, 0.5))]:
        got, amp = stretched_frequencies(base, dims, StretchConfig(*s))
        want, wamp = plain.stretched_frequencies(base, dims, dict(zip(("factor", "original", "fast", "slow"), s)))
        assert got == pytest.approx(want, rel=1e-14) and amp == pytest.approx(wamp, rel=1e-14)
    # inside a ramp the frequency lies strictly between the two
    got, _ = stretched_frequencies(10000.0, 64, StretchConfig(8.0, 512, 32.0, 1.0))
    plain_f = [10000.0 ** (-2 * i / 64) for i in range(32)]
    inside = [i for i in range(32) if plain_f[i] / 8.0 * 1.0001 < got[i] < plain_f[i] * 0.9999]
    assert inside and got[0] == plain_f[0] and got[31] == pytest.approx(plain_f[31] / 8.0)


# ----------------------------------------------------------------------------- chunks of long requests
def test_cut_long_requests():
    short, blocks, longs = cut_long_requests([0, 5, 6, 136, 200], [5, 1, 130, 64, 15], 64, 16)
    assert short.tolist() == [[0, 0, 5], [1, 5, 1], [4, 200, 15]]
    assert blocks.tolist() == [[2, 6, 64, 0], [2, 70, 64, 0], [2, 134, 2, 0], [3, 136, 64, 0]]
    assert longs.tolist() == [[2, 6, 130, 0], [3, 136, 64, 3]]
    short, blocks, longs = cut_long_requests([0], [3], 64, 16)
    assert short.shape == (1, 3) and blocks.shape == (0, 4) and longs.shape == (0, 4) and blocks.dtype == np.int32


# ----------------------------------------------------------------------------- the oracle's small functions
def test_plain_decayed_state_is_a_decayed_sum():
    torch.manual_seed(0)
    T, width, H, n, nv = 7, 5, 2, 3, 4
    m = {"heads": H, "dim": n, "vdim": nv, "decay": [0.5, 1.0]}
    w = {"q": torch.randn(H * n, width), "k": torch.randn(H * n, width), "v": torch.randn(H * nv, width),
         "g": torch.randn(H * nv, width), "norm": torch.rand(H * nv) + 0.5, "o": torch.eye(H * nv)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(T, width, dtype=torch.float64)
    got = plain.decayed_state_mixer(h, m, w, "", 1e-6)
    q, k = plain.silu(h @ w["q"].T).reshape(T, H, n), plain.silu(h @ w["k"].T).reshape(T, H, n)
    v = plain.silu(h @ w["v"].T).reshape(T, H, nv)
    o = torch.zeros(T, H, nv, dtype=torch.float64)
    for t in range(T):
        for a in range(H):
            for j in range(t + 1):
                o[t, a] += m["decay"][a] ** (t - j) * (q[t, a] @ k[j, a]) * v[j, a]
    want = plain.rms_norm(o.reshape(T, -1), w["norm"], 1e-6) * torch.sigmoid(h @ w["g"].T)
    assert torch.allclose(got, want, rtol=1e-12, atol=1e-12)
    # a state carried over: two halves equal the whole
    S = torch.zeros(H, n, nv, dtype=torch.float64)
    first = plain.decayed_state_mixer(h[:3], m, w, "", 1e-6, state=S)
    second = plain.decayed_state_mixer(h[3:], m, w, "", 1e-6, state=S)
    assert torch.allclose(torch.cat([first, second]), got, rtol=1e-12, atol=1e-12)


def test_plain_softmax_with_a_learned_sink_and_squashed_scores():
    q = torch.tensor([[[1.0, 0.0]], [[0.0, 2.0]]], dtype=torch.float64)          # [T=2, H=1, n=2]
    k = torch.tensor([[[1.0, 1.0]], [[0.5, -1.0]]], dtype=torch.float64)
    v = torch.tensor([[[1.0]], [[3.0]]], dtype=torch.float64)
    sink = torch.tensor([0.7], dtype=torch.float64)
    out = plain.softmax_attention(q, k, v, 0.5, sink=sink)
    s = torch.tensor([0.5 * 2.0, 0.5 * -2.0], dtype=torch.float64)                 # query 1 against keys 0 and 1
    e = torch.exp(s)
    assert float(out[1, 0, 0]) == pytest.approx(float((e[0] * 1.0 + e[1] * 3.0) / (e.sum() + math.exp(0.7))))
    assert float(out[0, 0, 0]) == pytest.approx(math.exp(0.5) / (math.exp(0.5) + math.exp(0.7)))
    capped = plain.softmax_attention(q * 100.0, k, v, 0.5, cap=2.0)
    s = 2.0 * torch.tanh(torch.tensor([100.0, -100.0], dtype=torch.float64) / 2.0)
    e = torch.exp(s)
    assert float(capped[1, 0, 0]) == pytest.approx(float((e[0] + 3.0 * e[1]) / e.sum()))
    # a window of one sees the token itself only
    alone = plain.softmax_attention(q, k, v, 0.5, window=1)
    assert alone[:, 0, 0].tolist() == [1.0, 3.0]


def test_plain_rotation_turns_halves_with_an_amplitude():
    v = torch.randn(3, 2, 10, dtype=torch.float64)
    sc = {"factor": 2.0, "original": 1.0, "fast": 1e3, "slow": 1e2}              # every pair but the first divided by two
    out = plain.turn_halves(v, [0, 5, 9], 100.0, 6, sc)
    amp = 0.1 * math.log(2.0) + 1.0
    assert torch.allclose(out[0, :, :6], v[0, :, :6] * amp) and torch.equal(out[:, :, 6:], v[:, :, 6:])
    a = 5 * 100.0 ** (-2.0 * 1 / 6) / 2.0                                          # pair (1, 4) at position 5
    assert torch.allclose(out[1, :, 1], amp * (v[1, :, 1] * math.cos(a) - v[1, :, 4] * math.sin(a)))
    assert torch.allclose(out[1, :, 4], amp * (v[1, :, 4] * math.cos(a) + v[1, :, 1] * math.sin(a)))


def test_plain_gelu_and_order():
    z = torch.linspace(-4, 4, 9, dtype=torch.float64)
    assert torch.allclose(plain.gelu_tanh(z), torch.nn.functional.gelu(z, approximate="tanh"))
    assert plain.run_order(ODD) == [(0, False), (1, True), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False), (4, False)]
