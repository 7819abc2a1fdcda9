"""Random configurations of the Sofudra decoder: `random_config(case)` is a pure function of the case number and draws
every size, the kinds and the order of the layers, which of them a loop takes in and how often, the windows and the
constants; each case runs whole and mixed with other requests on a small pool, in float32 and in bfloat16, against the
oracle.  The bfloat16 cases draw sizes in multiples of 8 (what the tensor-core products take).  The decayed states have
at least four values per head and decays of 0.3 and more: the norm behind a single value keeps its sign only, and with
a decay of nought a head's output is its value times q . k, of which the norm again keeps the sign, which rounding flips
near nought (a decay of nought runs in the tests of the kernels, in front of the norm)."""
import random

import pytest
import torch

import replay_lib as rl
from sofudra_helpers import (TOL_BF16, TOL_F32, attn, check_against_plain, config, decayed, gated, layer, make_model, par, poison,
                             rel_err, seeded_ids)

pytestmark = pytest.mark.gpu


def random_config(case: int, even: bool = False):
    rng = random.Random(2000 + case)
    unit = 8 if even else 1
    width = rng.choice([64, 128, 192]) if even else rng.randrange(24, 100)

    def head_sizes():
        kv = rng.choice([1, 1, 2, 3])
        heads = kv * rng.choice([1, 1, 2, 3, 4])
        dim = rng.choice([32, 64, 128]) if even else 2 * rng.randrange(2, 20)
        vdim = rng.choice([dim, dim, 16, 32, 64]) if even else rng.choice([dim, rng.randrange(1, 40)])
        return heads, kv, dim, vdim

    layers = []
    for _ in range(rng.randrange(1, 5)):
        heads, kv, dim, vdim = head_sizes()
        scale = rng.uniform(0.3, 2.0) / dim ** 0.5
        if rng.random() < 0.5:
            rot = rng.choice([dim, 2 * rng.randrange(1, dim // 2 + 1)])
            scaling = rng.choice([None, (rng.choice([1.0, 2.0, 3.7, 6.0]), rng.choice([16, 64, 512]),
                                         rng.choice([24.0, 4.0]), rng.choice([1.0, 0.5, 2.0]))])
            mixer = attn(heads, kv, dim, vdim, scale, window=rng.choice([1, 2, rng.randrange(3, 20), rng.randrange(20, 200)]),
                         rot=rot, base=rng.choice([10.0, 1000.0, 5e5]), scaling=scaling)
        else:
            dh = rng.randrange(1, 5)
            dn = rng.choice([16, 32, 64]) if even else rng.randrange(1, 40)
            dv = rng.choice([16, 32, 64]) if even else rng.randrange(4, 40)
            decay = [rng.choice([0.3, 1.0, rng.uniform(0.3, 0.999), rng.uniform(0.9, 0.9999)]) for _ in range(dh)]
            mixer = par(gated(heads, kv, dim, vdim, scale, rng.choice([1.0, 5.0, 30.0, 100.0])), decayed(dh, dn, dv, decay),
                        rng.uniform(0.5, 1.5), rng.uniform(0.5, 1.5))
        layers.append(layer(mixer, rng.choice([None, unit * rng.randrange(2, 30), unit * rng.randrange(2, 30)])))
    loop = None
    if rng.random() < 0.7:
        start = rng.randrange(0, len(layers))
        loop = (start, rng.randrange(start + 1, len(layers) + 1), rng.randrange(1, 4))
    cfg = config(rng.randrange(30, 300), width, rng.choice([1e-6, 1e-5, 1e-3]), layers, loop=loop,
                 embed_scale=rng.choice([1.0, 3.0, width ** 0.5]), mult=rng.choice([1.0, 0.3, 0.7]),
                 cap=rng.choice([None, 10.0, 30.0]))
    return cfg, rng.choice([4, 8, 16, 32, 64])


@pytest.mark.parametrize("case", range(12))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_configuration(model_root, case, dtype):
    cfg, page = random_config(case, even=(dtype == "bfloat16"))
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = make_model(model_root, f"random{case}", seed=case, dtype=stored, config_json=cfg)
    reqs = {f"r{i}": seeded_ids(n, cfg["vocab"], 7 * case + i) for i, n in enumerate([61, 18, 130, 40, 77])}
    mixed_steps, peak = rl.mixed(reqs, seed=case)
    from beglin_b200 import Engine
    results = {}
    for way, (steps, tokens) in {"whole": (rl.whole(reqs), 192), "mixed": (mixed_steps, peak)}.items():
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=max(tokens, page), page_size=page, max_requests=4, kv_split=64)
        poison(eng)
        results[way] = rl.run_in_process(eng, steps)
        eng.cache.check()
        check_against_plain(results[way], folder, reqs, TOL_F32 if dtype == "float32" else TOL_BF16)
    if dtype == "float32":
        for key, row in results["whole"].items():
            assert rel_err(results["mixed"][key], row) < 2 * TOL_F32, key      # (two roundings of their own)
