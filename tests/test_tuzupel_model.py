"""The Tuzupel decoder through the engine against the plain implementation: whole prompts, the same requests cut and
batched in four ways, single tokens from the first position on, long decoding over page, block, window and chunk borders,
decoding as a replayed graph, greedy generation through the scheduler, and the trace program."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import replay_lib as rl
from tuzupel_helpers import (CONFIGS, TOL_BF16, TOL_F32, check_against_plain, make_model, plain_logits, poison, rel_err,
                             seeded_ids)

pytestmark = pytest.mark.gpu

LENGTHS = {"odd": [70, 45, 100, 33, 120, 64], "sharp": [130, 33, 250, 97, 64, 180], "even": [150, 41, 300, 90, 65, 129]}


def requests_for(name):
    vocab = CONFIGS[name][0]["vocab"]
    return {f"r{i}": seeded_ids(n, vocab, 100 + i) for i, n in enumerate(LENGTHS[name])}


def engine_for(folder, dtype, max_tokens, page_size, kv_split=64, max_requests=4, **kw):
    from beglin_b200 import Engine
    e = Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, page_size=page_size, max_requests=max_requests,
                           kv_split=kv_split, **kw)
    poison(e)
    return e


def stored(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


@pytest.mark.parametrize("name,dtype", [("odd", "float32"), ("odd", "bfloat16"), ("even", "float32"), ("even", "bfloat16"),
                                        ("sharp", "float32")])
def test_four_ways_of_cutting(model_root, name, dtype):
    """Whole; the last 32 tokens one by one; portions down to two tokens; up to four live requests on a pool so
    small that pages and slots are used again.  Every way against the plain logits, and in float32 the four ways against
    one another within rounding (long portions walk the recurrence in chunks, single tokens one by one)."""
    folder = make_model(model_root, name, seed=11, dtype=stored(dtype))
    page = CONFIGS[name][1]
    reqs = requests_for(name)
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    mixed_steps, peak = rl.mixed(reqs, seed=5)
    longest = -(-max(LENGTHS[name]) // 64) * 64
    ways = {"whole": (rl.whole(reqs), longest), "tail": (rl.last_one_by_one(reqs), longest),
            "portions": (rl.portions(reqs), longest), "mixed": (mixed_steps, peak)}
    results = {}
    for way, (steps, max_tokens) in ways.items():
        eng = engine_for(folder, dtype, max_tokens, page)
        results[way] = rl.run_in_process(eng, steps)
        eng.cache.check()
        assert not eng.cache.live() and eng.cache.free_pages() == eng.cache.num_pages
        check_against_plain(results[way], folder, reqs, tol)
    if dtype == "float32":
        for way in ("tail", "portions", "mixed"):
            for key, row in results["whole"].items():
                assert rel_err(results[way][key], row) < 2 * TOL_F32, (way, key)


@pytest.mark.parametrize("name", ["odd", "even", "sharp"])
def test_first_tokens_one_by_one(model_root, name):
    """A request that starts with single tokens: the first positions of a sequence, where a window and a convolution reach
    back before the start, the only key is the token itself beside the sink, and the recurrence begins at nought."""
    folder = make_model(model_root, name, seed=11, dtype=torch.float32)
    ids = seeded_ids(9, CONFIGS[name][0]["vocab"], 9)
    eng = engine_for(folder, "float32", 64, CONFIGS[name][1])
    steps = [{"entries": [{"id": "x", "tokens": ids[:1], "want": [0]}]},
             {"entries": [{"id": "x", "tokens": ids[1:2], "want": [0]}]},
             {"entries": [{"id": "x", "tokens": ids[2:4], "want": [0, 1]}]},
             {"entries": [{"id": "x", "tokens": ids[4:5], "want": [0]}]},
             {"entries": [{"id": "x", "tokens": ids[5:9], "want": [0, 1, 2, 3]}], "end": ["x"]}]
    got = rl.run_in_process(eng, steps)
    check_against_plain(got, folder, {"x": ids}, TOL_F32)


def test_long_decoding_over_every_border(model_root):
    """700 positions over pages of 16 and splits of 64 keys under sharp softmaxes, in layers whose blocks of positions and
    windows hold 150 and 33 positions: a prompt in two portions that end inside a page, a split, a block and a chunk of the
    recurrence, then single tokens over their borders.  A key lost, taken from a wrong page, or let in from just outside a
    window or from the block before changes the logits altogether."""
    from tuzupel_helpers import CONFIGS as C
    folder = make_model(model_root, "sharp", seed=3, dtype=torch.float32)
    ids = seeded_ids(700, C["sharp"][0]["vocab"], 77)
    eng = engine_for(folder, "float32", 704, 16, kv_split=64)
    steps = [{"entries": [{"id": "a", "tokens": ids[:250], "want": list(range(250))}]},
             {"entries": [{"id": "a", "tokens": ids[250:637], "want": list(range(387))}]}]
    steps += [{"entries": [{"id": "a", "tokens": [ids[i]], "want": [0]}], "end": ["a"] if i == 699 else []}
              for i in range(637, 700)]
    got = rl.run_in_process(eng, steps)
    # a softmax that one key carries is ill-conditioned (the rounding of a score moves the weights themselves), so the
    # bound is some ten times the usual one, which a lost key breaks a hundredfold
    check_against_plain(got, folder, {"a": ids}, 5e-4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_as_a_graph_and_greedy_generation(model_root, dtype):
    """`Engine.generate` (scheduler, sampler, decoding steps replayed as graphs with padded rows) gives, for prompts of
    unequal lengths, the tokens that the plain implementation's argmax gives when it is fed its own choices."""
    name = "even"
    folder = make_model(model_root, name, seed=21, dtype=stored(dtype))
    vocab = CONFIGS[name][0]["vocab"]
    prompts = [seeded_ids(n, vocab, 50 + n) for n in (37, 5, 90)]
    new = 12
    from beglin_b200 import Engine
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=512, page_size=16, max_requests=4)
    outs = eng.generate(prompts, max_new_tokens=new, stop_ids=())
    for p, out in zip(prompts, outs):
        assert len(out) == new
        ids = list(p)
        for k, tok in enumerate(out):
            want = plain_logits(folder, ids)[-1]
            top2 = torch.topk(want, 2).values
            if dtype == "bfloat16" and float(top2[0] - top2[1]) < 0.1 * float(want.abs().max()):
                break                                   # a close call in a rounded format: what follows is another text
            assert int(torch.argmax(want)) == tok, (len(p), k)
            ids.append(tok)


def test_trace_program(model_root, tmp_path):
    """bin/trace_run on a Tuzupel folder: the architecture is picked from config.json, the steps come on standard input,
    the logits land in files."""
    name = "odd"
    folder = make_model(model_root, name, seed=11, dtype=torch.float32)
    reqs = {k: v for k, v in list(requests_for(name).items())[:3]}
    steps, peak = rl.mixed(reqs, seed=2)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", str(out), "--max-tokens", str(peak), "--page-size", "16"],
                       input="\n".join(json.dumps(s) for s in rl.number(steps)) + "\n", text=True, capture_output=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    vocab = CONFIGS[name][0]["vocab"]
    held = {}
    for i, s in enumerate(steps):
        rows = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, vocab)
        r = 0
        for e in s["entries"]:
            start = held.get(e["id"], 0)
            want = plain_logits(folder, reqs[e["id"]])
            for w in e["want"]:
                assert rel_err(torch.from_numpy(rows[r].copy()), want[start + w]) < TOL_F32 * float(want.abs().max() / want[start + w].abs().max())
                r += 1
            held[e["id"]] = start + len(e["tokens"])
        assert r == rows.shape[0]


def test_command_line_greedy(model_root, tmp_path):
    """`qwen_infer greedy N` on a Tuzupel folder: the registry picks the architecture from config.json, and the
    tokens are those of Engine.generate."""
    folder = make_model(model_root, "even", seed=4, dtype=torch.bfloat16)
    prompt = seeded_ids(21, CONFIGS["even"][0]["vocab"], 5)
    path = tmp_path / "prompt.i32"
    np.asarray(prompt, dtype="<i4").tofile(path)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, QWEN_BASE=folder, QWEN_PROMPT=str(path), QWEN_SAFETENSORS_MAXSEQ="128", QWEN_DTYPE="fp32")
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "qwen_infer"), "greedy", "6"], env=env, capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("greedy:")][0]
    toks = [int(t) for t in line.split(":")[1].split()]
    from beglin_b200 import Engine
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=128, max_requests=1)
    assert toks == eng.generate([prompt], max_new_tokens=6, stop_ids=())[0]


def test_slots_and_pages_used_again(model_root):
    """Two state slots and five pages of 16 for six requests that come one after the other or two at a time: every
    request's slot and pages were another request's before (NaN was in all of them at the start)."""
    name = "odd"
    folder = make_model(model_root, name, seed=11, dtype=torch.float32)
    vocab = CONFIGS[name][0]["vocab"]
    reqs = {f"q{i}": seeded_ids(n, vocab, 300 + i) for i, n in enumerate([30, 40, 25, 33, 16, 38])}
    eng = engine_for(folder, "float32", 80, 16, max_requests=2)
    order = list(reqs)
    steps = []
    for a, b in zip(order[0::2], order[1::2]):
        ia, ib = reqs[a], reqs[b]
        steps.append({"entries": [{"id": a, "tokens": ia[:7], "want": list(range(7))}]})
        steps.append({"entries": [{"id": a, "tokens": ia[7:], "want": list(range(len(ia) - 7))},
                                  {"id": b, "tokens": ib[:3], "want": [0, 1, 2]}], "end": [a]})
        steps.append({"entries": [{"id": b, "tokens": ib[3:], "want": list(range(len(ib) - 3))}], "end": [b]})
    got = rl.run_in_process(eng, steps)
    eng.cache.check()
    check_against_plain(got, folder, reqs, TOL_F32)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_portion_replayed_as_a_graph(model_root, dtype):
    """A portion of 300 tokens of one request in a shape that came before is replayed as a CUDA graph (the engine's own
    rule): three requests of that shape one after the other, the third behind a first portion of its own so that the graph
    runs at other positions, windows, blocks and chunk states than it was captured at; every one against the plain logits."""
    name = "even"
    folder = make_model(model_root, name, seed=31, dtype=stored(dtype))
    vocab = CONFIGS[name][0]["vocab"]
    reqs = {"a": seeded_ids(300, vocab, 1), "b": seeded_ids(300, vocab, 2), "c": seeded_ids(341, vocab, 3)}
    want = [0, 100, 299]
    eng = engine_for(folder, dtype, 384, 16, max_requests=2)
    steps = [{"entries": [{"id": "a", "tokens": reqs["a"], "want": want}], "end": ["a"]},
             {"entries": [{"id": "b", "tokens": reqs["b"], "want": want}], "end": ["b"]},
             {"entries": [{"id": "c", "tokens": reqs["c"][:41], "want": [40]}]},
             {"entries": [{"id": "c", "tokens": reqs["c"][41:], "want": want}], "end": ["c"]}]
    got = rl.run_in_process(eng, steps)
    assert eng.portions.replays >= 2
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    for rid, ids in reqs.items():
        full = plain_logits(folder, ids)
        for (r, p), row in got.items():
            if r == rid:
                assert rel_err(row, full[p]) < tol * float(full.abs().max() / full[p].abs().max()), (rid, p)
