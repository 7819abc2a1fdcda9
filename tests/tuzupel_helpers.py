"""Configurations, lively random weights and comparison helpers for the tests of the Tuzupel decoder.

The configurations differ from one another and from layer to layer in every size: one to four query heads per kv head,
values narrower than, as wide as and wider than keys, head sizes that are no powers of two, blocks of positions and
windows shorter than a page and of several pages, rotation of a part of a head and of all of it, rescaled frequencies
whose bands begin at, inside and behind the head's frequencies, one to four lanes or a plain residual, recurrences of
one to five parts with convolutions of one to five taps, experts with and without identity experts, a shared expert
and a choice bias, one to three experts per token, layers without a feed-forward.
"""
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "plain"))
import tuzupel_plain as plain  # noqa: E402

# Angles are float by design: at position p a pair of frequency f turns by an angle that carries a rounding of 2^-24 p f,
# which a rotation of whole heads at a small base (every pair turning fast) shows in the logits.
TOL_F32 = 5e-5
TOL_BF16 = 4e-2
# Random configurations in bfloat16: three recurrences in a row behind a norm with a large eps reach 0.066 where the same
# folder in float32 stays at 1e-6; a fault of a kernel shows as an error of the size of the logits themselves.
TOL_BF16_RANDOM = 8e-2
ROUTE_DIMS = 4      # features of the residual that belong to the routers alone in a model with decisive routers


def attn(heads, kv_heads, dim, vdim, scale, block=None, rot=None, base=10000.0, scaling=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if block is not None:
        m["mask"] = {"size": block}
    if rot:
        m["rot"] = {"base": base, "dims": rot}
        if scaling is not None:
            factor, low, high, original = scaling
            m["rot"]["scaling"] = {"factor": factor, "low": low, "high": high, "original": original}
    return "attention", m


def lat(heads, dim, vdim, kv_rank, scale, window=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return "latent_attention", m


def rec(width, blocks, conv):
    return "rglru", {"width": width, "blocks": blocks, "conv": conv}


def moe(ff, limit, experts, top, scale=1.0, identity=0, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff, "limit": limit},
         "router": {"experts": experts, "identity": identity, "scale": scale, "top": top}}
    if shared is not None:
        f["shared"] = {"ff": shared[0], "limit": shared[1]}
    return f


def layer(mixer, mlp=None):
    return {"type": mixer[0], "mixer": mixer[1], "mlp": mlp}


def config(vocab, width, eps, layers, streams=None, cap=None):
    out = {"architecture": "Tuzupel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams is not None:
        out["streams"] = streams
    if cap is not None:
        out["logit_softcap"] = cap
    return out


# odd sizes everywhere; every layer differs from the others; three lanes
ODD = config(211, 72, 1e-6, [
    layer(attn(3, 1, 10, 6, 0.4, block=13, rot=8, base=100.0, scaling=(2.5, 1.0, 4.0, 64)), moe(20, 1.5, 5, 2, 1.7, identity=2, shared=(28, 3.0))),
    layer(rec(36, 3, 4), moe(12, 2.0, 3, 1, 0.8)),
    layer(lat(4, 12, 9, 20, 0.3, window=17), moe(9, 7.0, 4, 3, 2.5, identity=1)),
    layer(attn(4, 2, 12, 12, 0.3, block=40, rot=12, base=10.0)),                                        # no feed-forward
    layer(rec(25, 1, 1), moe(31, 0.7, 6, 2, 1.0, shared=(5, 1.0))),
    layer(lat(2, 6, 14, 7, 0.5), moe(8, 2.0, 2, 2, 1.0, identity=3)),                                   # no window
], streams=3, cap=20.0)
# sharp attention: large score scales make every softmax pick out single keys; one plain residual, no squashed logits
SHARP = config(150, 64, 1e-5, [
    layer(attn(4, 2, 16, 8, 2.5, block=150, rot=8, base=1000.0, scaling=(4.0, 0.5, 8.0, 128)), moe(24, 2.0, 4, 2, 1.0, identity=1)),
    layer(lat(2, 24, 16, 32, 2.0, window=33), moe(16, 2.0, 4, 1, 2.0, shared=(16, 2.0))),
    layer(rec(48, 2, 3)),
    layer(attn(2, 1, 24, 16, 2.0, block=33, rot=24, base=300.0), moe(8, 2.0, 3, 2, 1.0)),
])
# sizes in multiples of 64: in bfloat16 the products run this package's tensor-core kernels; two lanes
EVEN = config(320, 128, 1e-5, [
    layer(attn(4, 2, 64, 64, 0.125, block=80, rot=32, base=10000.0, scaling=(4.0, 1.0, 4.0, 256)), moe(64, 2.0, 8, 2, 2.0, identity=2, shared=(128, 2.0))),
    layer(lat(4, 64, 64, 64, 0.125, window=70), moe(128, 3.0, 4, 1, 1.0)),
    layer(rec(128, 2, 4), moe(64, 2.0, 8, 3, 1.5, identity=1, shared=(64, 4.0))),
    layer(attn(2, 2, 128, 128, 0.09, block=200, rot=64, base=200000.0), moe(64, 2.0, 4, 2, 1.0)),
    layer(lat(2, 128, 128, 96, 0.09, window=200)),
    layer(attn(8, 2, 32, 64, 0.18, rot=16, base=1000.0, scaling=(2.0, 2.0, 16.0, 64)), moe(192, 1.0, 2, 2, 1.0, identity=2)),
], streams=2, cap=12.0)
CONFIGS = {"odd": (ODD, 8), "sharp": (SHARP, 16), "even": (EVEN, 16)}        # name -> (config, page size)


def lively_tensors(cfg_json, seed, dtype, decisive=False):
    """Random weights under which every mechanism matters: matrices of unit gain, norm weights spread around their
    centre, sinks and corrections of the size of the scores they meet, decays between a few and many tokens.  The names
    and shapes come from the framework's loader; the values are drawn here.

    `decisive`: for runs in a rounded number format, where a router that reads rounded rows could choose another expert
    than the oracle on a close call.  The last ROUTE_DIMS features of the residual then belong to the routers alone: the
    embedding marks one of them per token, no sublayer's last matrix writes there (an identity expert only rescales what
    is there), and a router reads nothing else, through weights that are spaced evenly: the order of a token's scores is
    the order of one column of the router, whatever the rounding of the row.  There is no choice bias then."""
    from beglin_b200.config import load_config
    from beglin_b200.weights import expected_tensors
    arch, cfg = load_config(dict(cfg_json))
    spec = arch.build_spec(cfg)
    g = torch.Generator().manual_seed(seed)
    out = {}
    n = cfg_json.get("streams") or 1
    for name, role in expected_tensors(spec).items():
        shape = tuple(role.shape)
        r = lambda *s: torch.randn(*s, generator=g)
        last = name.rsplit(".", 1)[-1]
        if name == "embed":
            t = r(*shape) * 0.5
            if decisive:
                t[:, -ROUTE_DIMS:] = 0.0
                t[torch.arange(shape[0]), shape[1] - ROUTE_DIMS + torch.arange(shape[0]) % ROUTE_DIMS] = 2.0
        elif last == "sink":
            t = r(*shape) * 1.5
        elif last == "correction":
            t = torch.zeros(shape) if decisive else r(*shape) * 0.1
        elif last == "router":
            t = r(*shape) * (2.0 / shape[1] ** 0.5)
            if decisive:
                t = torch.zeros(shape)
                for k in range(ROUTE_DIMS):
                    t[:, shape[1] - ROUTE_DIMS + k] = 0.3 * (1 + torch.randperm(shape[0], generator=g)).float()
        elif last == "lam":
            t = -6.0 * torch.rand(*shape, generator=g)
        elif last == "b":
            t = r(*shape) * 0.5
        elif last == "conv":
            t = r(*shape) * 0.5
        elif name.endswith(".norm1") or name.endswith(".norm2") or name == "final.norm":
            t = 0.2 * r(*shape)                     # stored around zero
        elif last == "norm":
            t = 1.0 + 0.2 * r(*shape)               # plain weights
        elif ".hc" in name and last == "in":
            t = 0.9 / n + 0.2 * r(*shape)
        elif ".hc" in name and last == "out":
            t = 0.8 + 0.3 * r(*shape)
        elif ".hc" in name and last == "mix":
            t = 0.8 * torch.eye(shape[0]) + 0.15 * r(*shape)
        else:
            t = r(*shape) * (1.2 / shape[-1] ** 0.5)
            if decisive and (last in ("o", "down")):
                t[-ROUTE_DIMS:] = 0.0
        out[name] = t.to(dtype)
    return out


def write_model(folder, cfg, tensors):
    from beglin_b200.weights import write_safetensors
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    return folder


def make_model(root, name, seed=0, dtype=torch.float32, config_json=None, decisive=None):
    """Write a model folder with lively random weights under `root` and return its path.  A folder stored in bfloat16
    gets decisive routers unless told otherwise."""
    cfg = CONFIGS[name][0] if config_json is None else config_json
    decisive = (dtype != torch.float32) if decisive is None else decisive
    folder = os.path.join(str(root), f"tuzupel_{name}_{seed}_{str(dtype).split('.')[-1]}_{int(decisive)}")
    if not os.path.exists(os.path.join(folder, "model.safetensors")):
        write_model(folder, cfg, lively_tensors(cfg, seed, dtype, decisive))
    return folder


_CACHE = {}


def plain_logits(folder, ids):
    """float64 logits [T, vocab] of the whole sequence from the plain implementation."""
    if folder not in _CACHE:
        _CACHE[folder] = plain.read_folder(folder, torch.float64)
    key = (folder, tuple(ids))
    if key not in _CACHE:
        cfg, w = _CACHE[folder]
        _CACHE[key] = plain.forward(cfg, w, list(ids))
    return _CACHE[key]


def rel_err(got, want):
    want = want.to(torch.float64).cpu()
    got = got.to(torch.float64).cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


def seeded_ids(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def check_against_plain(got, folder, reqs, tol):
    """got: {(request, position): logits row}; every position of every request against the plain logits."""
    worst = 0.0
    for rid, ids in reqs.items():
        want = plain_logits(folder, ids)
        rows = torch.stack([got[(rid, p)] for p in range(len(ids))])
        assert torch.isfinite(rows).all(), rid
        err = rel_err(rows, want)
        if err > tol:
            per_pos = (rows.double() - want).abs().max(dim=1).values / want.abs().max()
            first = int((per_pos > tol).nonzero()[0])
            raise AssertionError(f"{rid}: relative error {err:.3g} > {tol:g}; first wrong position {first} of {len(ids)}")
        worst = max(worst, err)
    return worst


def poison(engine):
    """NaN in every page and state slot: a read of something that was never written, or of what an earlier request
    left, shows."""
    for g in engine.cache.kv_groups:
        g.device_pool.fill_(float("nan"))
    for g in engine.cache.state_groups:
        g.slab.fill_(float("nan"))
