"""Configurations, lively random weights and comparison helpers for the tests of the Sofudra decoder.

The configurations differ from one another and from layer to layer in every size: one to four query heads per kv head,
values narrower than, as wide as and wider than keys, head sizes that are no powers of two, windows shorter than a page
and of several pages, rotation of a part of a head and of all of it, stretched frequencies with ramps that begin at,
inside and behind the head, decays from 0 to nearly 1, loops that begin at the first layer, in the middle, or are absent,
attention layers inside a loop and parallel layers outside, layers without a feed-forward.
"""
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "plain"))
import sofudra_plain as plain  # noqa: E402

TOL_F32 = 3e-5
TOL_BF16 = 4e-2


def attn(heads, kv_heads, dim, vdim, scale, window=None, rot=None, base=10000.0, scaling=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"base": base, "dims": rot}
        if scaling is not None:
            factor, original, fast, slow = scaling
            m["rot"]["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    return m


def gated(heads, kv_heads, dim, vdim, scale, softcap):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap}


def decayed(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def par(left, right, left_scale=1.0, right_scale=1.0):
    return {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}


def layer(mixer, ff=None):
    return {"type": "parallel" if "left" in mixer else "attention", "mixer": mixer,
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(vocab, width, eps, layers, loop=None, embed_scale=1.0, mult=1.0, cap=None):
    out = {"architecture": "Sofudra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale},
           "residual_mult": mult, "layers": layers}
    if cap is not None:
        out["logit_softcap"] = cap
    if loop is not None:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


# odd sizes everywhere; every layer differs from the others; the loop takes in an attention layer and a parallel one
ODD = config(211, 72, 1e-6, [
    layer(par(gated(3, 1, 10, 6, 0.4, 5.0), decayed(3, 6, 10, [0.5, 0.9, 0.99]), 0.7, 1.3), 100),
    layer(attn(4, 2, 12, 12, 0.3, window=13, rot=8, base=100.0, scaling=(2.5, 64, 4.0, 0.5)), 60),
    layer(par(gated(2, 2, 16, 24, 0.25, 50.0), decayed(1, 14, 5, [0.97]), 1.5, 0.5)),                # no feed-forward
    layer(attn(3, 3, 6, 2, 0.5, window=40, rot=6, base=10.0), 33),                                      # no stretching
    layer(attn(4, 1, 8, 14, 0.35, window=7, rot=4, base=50.0, scaling=(3.0, 16, 2.0, 1.0))),
], loop=(1, 3, 3), embed_scale=4.0, mult=0.4, cap=20.0)
# sharp attention: large score scales make every softmax pick out single keys; decays close to one keep far tokens
SHARP = config(150, 64, 1e-5, [
    layer(attn(4, 2, 16, 8, 2.5, window=150, rot=8, base=1000.0, scaling=(4.0, 128, 8.0, 1.0)), 96),
    layer(par(gated(2, 1, 24, 16, 2.0, 25.0), decayed(2, 8, 8, [0.999, 1.0]), 1.0, 1.0), 48),
    layer(attn(2, 1, 24, 16, 2.0, window=33, rot=24, base=300.0), 40),
], loop=(0, 2, 2), embed_scale=2.0, mult=0.5)
# sizes in multiples of 64: in bfloat16 the products run this package's tensor-core kernels; no loop
EVEN = config(320, 128, 1e-5, [
    layer(attn(4, 2, 64, 64, 0.125, window=80, rot=32, base=10000.0, scaling=(4.0, 256, 16.0, 2.0)), 256),
    layer(par(gated(4, 1, 64, 32, 0.125, 20.0), decayed(2, 64, 64, [0.9, 0.995]), 1.1, 0.9), 192),
    layer(par(gated(2, 2, 128, 128, 0.09, 10.0), decayed(4, 32, 16, [0.6, 0.8, 0.95, 0.99]), 0.8, 1.2), 128),
    layer(attn(8, 2, 32, 64, 0.18, window=200, rot=16, base=1000.0)),
], embed_scale=8.0, mult=0.35, cap=12.0)
CONFIGS = {"odd": (ODD, 8), "sharp": (SHARP, 16), "even": (EVEN, 16)}        # name -> (config, page size)


def lively_tensors(cfg_json, seed, dtype):
    """Random weights under which every mechanism matters: matrices of unit gain, norm weights spread around one, biases
    and sinks of the size of the scores.  The names and shapes come from the framework's loader; the values are drawn
    here."""
    from beglin_b200.config import load_config
    from beglin_b200.weights import expected_tensors
    arch, cfg = load_config(dict(cfg_json))
    spec = arch.build_spec(cfg)
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, role in expected_tensors(spec).items():
        shape = tuple(role.shape)
        r = lambda *s: torch.randn(*s, generator=g)
        if name == "embed":
            t = r(*shape) * 0.5
        elif name.endswith(".sink"):
            t = r(*shape) * 1.5
        elif name.endswith(".b"):
            t = r(*shape) * 0.5
        elif len(shape) == 1:                       # norm weights
            t = 1.0 + 0.2 * r(*shape)
        else:
            t = r(*shape) * (1.2 / shape[1] ** 0.5)
        out[name] = t.to(dtype)
    return out


def write_model(folder, cfg, tensors):
    from beglin_b200.weights import write_safetensors
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    return folder


def make_model(root, name, seed=0, dtype=torch.float32, config_json=None):
    """Write a model folder with lively random weights under `root` and return its path."""
    cfg = CONFIGS[name][0] if config_json is None else config_json
    folder = os.path.join(str(root), f"sofudra_{name}_{seed}_{str(dtype).split('.')[-1]}")
    if not os.path.exists(os.path.join(folder, "model.safetensors")):
        write_model(folder, cfg, lively_tensors(cfg, seed, dtype))
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
