"""Random configurations of the Tuzupel decoder: `random_config(case)` is a pure function of the case number and draws
every size, the kinds and the order of the layers, the number of lanes, the blocks of positions and windows, the experts'
numbers and constants; each case runs whole and mixed with other requests on a small pool, in float32 and in bfloat16,
against the oracle.  The bfloat16 cases draw sizes in multiples of 8 (what the tensor-core products take) and routers
that no rounding can turn (see `lively_tensors`)."""
import random

import pytest
import torch

import replay_lib as rl
from tuzupel_helpers import (TOL_BF16_RANDOM, TOL_F32, attn, check_against_plain, config, lat, layer, make_model, moe, poison, rec,
                             rel_err, seeded_ids)

pytestmark = pytest.mark.gpu


def random_config(case: int, even: bool = False):
    rng = random.Random(3000 + case)
    unit = 8 if even else 1
    width = rng.choice([64, 128, 192, 200, 320]) if even else rng.randrange(24, 100)

    def mixer():
        kind = rng.choice(["attention", "latent_attention", "rglru"])
        if kind == "attention":
            kv = rng.choice([1, 1, 2, 3])
            heads = kv * rng.choice([1, 1, 2, 3, 4])
            dim = rng.choice([32, 64, 128, 48, 80, 96]) if even else 2 * rng.randrange(2, 20)
            vdim = rng.choice([dim, dim, 16, 32, 64, 40]) if even else rng.choice([dim, rng.randrange(1, 40)])
            rot = rng.choice([None, dim, 2 * rng.randrange(1, dim // 2 + 1)])
            scaling = rng.choice([None, (rng.choice([1.0, 2.0, 3.7, 8.0]), rng.choice([1.0, 0.5, 2.0]), rng.choice([4.0, 24.0]),
                                         rng.choice([16, 64, 512]))])
            return attn(heads, kv, dim, vdim, rng.uniform(0.3, 2.0) / dim ** 0.5,
                        block=rng.choice([None, 1, 2, rng.randrange(3, 20), rng.randrange(20, 200)]), rot=rot,
                        base=rng.choice([10.0, 1000.0, 5e5]), scaling=scaling)
        if kind == "latent_attention":
            heads = rng.randrange(1, 6)
            dim = rng.choice([32, 64, 128, 48, 24]) if even else rng.randrange(3, 40)
            vdim = rng.choice([dim, 16, 64, 40]) if even else rng.randrange(1, 40)
            rank = rng.choice([32, 64, 96, 160, 48, 200]) if even else rng.randrange(2, 50)
            return lat(heads, dim, vdim, rank, rng.uniform(0.3, 2.0) / dim ** 0.5,
                       window=rng.choice([None, 1, 2, rng.randrange(3, 20), rng.randrange(20, 200)]))
        blocks = rng.randrange(1, 6)
        return rec(blocks * (unit * rng.randrange(1, 6) if even else rng.randrange(1, 24)), blocks, rng.randrange(1, 6))

    def feed_forward():
        if rng.random() < 0.2:
            return None
        experts, identity = rng.randrange(1, 9), rng.choice([0, 0, 1, 3])
        shared = rng.choice([None, (unit * rng.randrange(1, 20), rng.choice([0.5, 2.0, 4.0]))])
        return moe(unit * rng.randrange(1, 20), rng.choice([0.5, 2.0, 4.0]), experts, rng.randrange(1, min(experts + identity, 4) + 1),
                   rng.choice([1.0, 2.5, 0.4]), identity=identity, shared=shared)

    layers = [layer(mixer(), feed_forward()) for _ in range(rng.randrange(1, 6))]
    cfg = config(rng.randrange(30, 300), width, rng.choice([1e-6, 1e-5, 1e-3]), layers, streams=rng.choice([None, 1, 2, 3, 4]),
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
        check_against_plain(results[way], folder, reqs, TOL_F32 if dtype == "float32" else TOL_BF16_RANDOM)
    if dtype == "float32":
        for key, row in results["whole"].items():
            assert rel_err(results["mixed"][key], row) < 2 * TOL_F32, key      # (two roundings of their own)
