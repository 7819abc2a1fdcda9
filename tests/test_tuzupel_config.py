"""The Tuzupel configuration on the CPU: the keys it reads, what it refuses, the description it builds, what the cache
manager is asked for, and the pages a block of positions gives back."""
import pytest

from tuzupel_helpers import CONFIGS, attn, config, lat, layer, rec


def load(cfg):
    from beglin_b200.config import load_config
    return load_config(dict(cfg))


def test_every_size_and_constant_is_read_from_the_configuration():
    arch, cfg = load(CONFIGS["odd"][0])
    assert arch.name == "Tuzupel" and cfg.lanes == 3 and cfg.logit_softcap == 20.0 and cfg.norm_eps == 1e-6
    spec = arch.build_spec(cfg)
    assert spec.lanes == 3 and spec.final_norm.offset == 1.0 and len(spec.layers) == 6
    a, r, l = spec.layers[0], spec.layers[1], spec.layers[2]
    assert a.block == "lanes_prenorm" and spec.layers[3].block == "lanes_prenorm_mixer"
    assert (a.mixer.n_heads, a.mixer.n_kv_heads, a.mixer.head_dim, a.mixer.v_head_dim, a.mixer.block, a.mixer.window) == (3, 1, 10, 6, 13, None)
    assert a.mixer.sink == "learned" and a.mixer.qk_norm == "head" and a.mixer.position.pairing == "interleaved"
    assert len(a.mixer.position.frequencies) == 4 and a.mixer.scale == 0.4
    f = a.feed_forward
    assert (f.experts, f.identity, f.top, f.route_scale, f.limit, f.intermediate) == (5, 2, 2, 1.7, 1.5, 20)
    assert f.router_activation == "softmax" and f.choice_bias and (f.shared.intermediate, f.shared.limit) == (28, 3.0)
    assert (r.mixer.width, r.mixer.blocks, r.mixer.conv, r.mixer.decay_scale) == (36, 3, 4, 8.0) and r.feed_forward.shared is None
    assert (l.mixer.kv_rank, l.mixer.window, l.mixer.q_rank, l.mixer.rot_dim, l.mixer.gated) == (20, 17, None, 0, False)
    assert spec.layers[5].mixer.window is None
    assert a.names["mixer_link.mix"] == "l0.hc1.mix" and a.names["feed_forward.router.bias"] == "l0.mlp.correction"
    assert r.names["mixer.gate_r.weight"] == "l1.mix.ra" and l.names["mixer.kv_down.norm"] == "l2.mix.dkv.norm"


def test_a_plain_residual_without_streams_and_a_folder_without_correction():
    arch, cfg = load(CONFIGS["sharp"][0])
    spec = arch.build_spec(cfg)
    assert spec.lanes == 0 and spec.layers[0].block == "prenorm" and spec.layers[2].block == "prenorm_mixer"
    assert spec.logit_softcap == 0.0
    from beglin_b200.config import load_config
    names = ["l0.mlp.router"]
    _, cfg2 = load_config(dict(CONFIGS["sharp"][0]), tensor_names=names)
    assert not arch.build_spec(cfg2).layers[0].feed_forward.choice_bias
    assert cfg.to_json_dict()["layers"][1]["mixer"]["mask"] == {"size": 33}
    again = load(cfg.to_json_dict())[1]
    assert again == cfg


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="conv"), "not known"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=2), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=11), "even"),
    (lambda c: c["layers"][1]["mixer"].update(blocks=5), "equal parts"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][0]["mlp"]["expert"].update(limit=0.0), "positive"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not known"),
    (lambda c: c.update(streams=9), "streams"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_what_is_refused(change, message):
    import copy
    from beglin_b200.config import ConfigError
    cfg = copy.deepcopy(CONFIGS["odd"][0])
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        load(cfg)


def test_cache_needs_and_pages_given_back_in_front_of_the_newest_block():
    from beglin_b200.cache.manager import CacheManager
    from beglin_b200.parts import registry
    from beglin_b200.parts.cache_need import FixedStateNeed, PagedKVNeed, PagedLatentNeed
    cfg = config(50, 32, 1e-5, [layer(attn(2, 1, 8, 4, 0.3, block=40)), layer(lat(2, 8, 8, 12, 0.3, window=20)), layer(rec(10, 2, 3)),
                                layer(attn(2, 2, 8, 8, 0.3))])
    arch, c = load(cfg)
    spec = arch.build_spec(c)
    needs = []
    for l in spec.layers:
        for _, family, cls, pspec in registry.layer_slots(l):
            if family == "mixer":
                needs.append(cls.cache_need(pspec, None) if getattr(cls, "cache_need_takes_context", False) else cls.cache_need(pspec))
    assert needs[0] == PagedKVNeed(1, 8, None, 4, 40) and needs[1] == PagedLatentNeed(12, 20)
    assert needs[2] == FixedStateNeed((30,), "float32") and needs[3] == PagedKVNeed(2, 8, None, None, None)
    m = CacheManager(needs, page_size=16, num_pages=12, max_requests=2)
    m.add_request("a")
    m.reserve([("a", 100)])
    m.commit([("a", 100)])
    free_before = [g.pool.num_free for g in m.kv_groups]
    m.reserve([("a", 101)])            # the query at 100 stands in the block [80, 120): pages 0..4 of the block group go back;
    m.commit([("a", 101)])             # its window of 20 begins at 81: pages 0..4 of the window group too; the last group keeps all
    gave = [g.pool.num_free - f for g, f in zip(m.kv_groups, free_before)]
    assert gave == [5, 5, 0]
    m.check()
    m.release("a")
    assert all(g.pool.num_free == 12 for g in m.kv_groups)
