"""The Sofudra decoder through the engine against the plain implementation: whole prompts, the same requests cut and
batched in four ways, single tokens from the first position on, long decoding over page, chunk and window borders,
attention that picks out single keys at the edges of a window and far back, a sink that carries a softmax, states that
keep the first tokens, decoding as a replayed graph, greedy generation through the scheduler, the command line and the
trace program."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import replay_lib as rl
from sofudra_helpers import (CONFIGS, TOL_BF16, TOL_F32, attn, check_against_plain, config, decayed, gated, layer, make_model,
                             par, plain, plain_logits, poison, rel_err, seeded_ids, write_model)

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
    small that pages are used again.  Every way against the plain logits, and in float32 the four ways against one
    another within rounding (long portions sum the decayed state in chunks, single tokens one by one)."""
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
    """A request that starts with single tokens: the first positions of a sequence, where a window reaches back before
    the start, the only key is the token itself beside the sink, and the state begins at nought."""
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


def test_far_keys_and_window_edges_under_sharp_attention(model_root):
    """700 positions over pages of 16 and splits of 64 keys, with score scales under which a softmax is carried by one
    or two keys, in layers with windows of 150 and 33 positions, one that sees everything, and states whose decays are
    0.999 and 1: a key lost, taken from a wrong page, or let in from just outside a window changes the logits
    altogether.  The prompt ends inside a page, a split and a chunk; single tokens follow over their borders."""
    folder = make_model(model_root, "sharp", seed=3, dtype=torch.float32)
    ids = seeded_ids(700, CONFIGS["sharp"][0]["vocab"], 77)
    want = plain_logits(folder, ids)
    eng = engine_for(folder, "float32", 704, 16, kv_split=64)
    steps = [{"entries": [{"id": "a", "tokens": ids[:250], "want": list(range(250))}]},
             {"entries": [{"id": "a", "tokens": ids[250:637], "want": list(range(387))}]}]
    steps += [{"entries": [{"id": "a", "tokens": [ids[i]], "want": [0]}], "end": ["a"] if i == 699 else []}
              for i in range(637, 700)]
    got = rl.run_in_process(eng, steps)
    # a softmax that one key carries is ill-conditioned (the rounding of a score moves the weights themselves), so the
    # bound is some ten times the usual one, which a lost key breaks a hundredfold
    tol = 5e-4
    check_against_plain(got, folder, {"a": ids}, tol)
    # the test means something: other tokens at positions 3 to 8 (which only the attention without a window and the
    # states see from afar) change the logits 690 positions later by far more than the tolerance
    other = list(ids)
    other[3:9] = [(t + 1) % CONFIGS["sharp"][0]["vocab"] for t in ids[3:9]]
    moved = rel_err(plain_logits(folder, other)[690:], want[690:])
    assert moved > 20 * tol, moved


# two attention layers only: every layer has a window, and rotation covers a part of the head so that a direction in
# the features behind it is the same at every position
WINDOWED = config(90, 48, 1e-5, [
    layer(attn(2, 1, 12, 10, 1.0, window=21, rot=4, base=40.0, scaling=(2.0, 32, 4.0, 1.0)), 40),
    layer(attn(3, 3, 8, 4, 1.0, window=64, rot=8, base=40.0), 24),
], mult=0.5)


def standout_model(model_root, dtype):
    """WINDOWED with weights under which ONE key stands out in the first layer: every token's queries point along the
    key of one token id, in the features that are not rotated.  (The norms of queries and keys keep directions only, so
    a key cannot be made long; what stands out is the direction that the queries share.)"""
    base = make_model(model_root, "windowed", seed=5, dtype=stored(dtype), config_json=WINDOWED)
    cfg, w = plain.read_folder(base, torch.float64)
    special, width, dimq, rot = 7, WINDOWED["width"], 12, 4
    tensors = {n: t.clone() for n, t in w.items()}
    u = torch.ones(width, dtype=torch.float64) / width ** 0.5
    tensors["embed"] += 3.0 * u                                    # every token is aligned with u
    tensors["l0.norm1"][:] = 1.0
    tensors["l0.mix.k"] -= torch.outer(tensors["l0.mix.k"] @ u, u)  # keys do not see u: their directions differ by token
    h = plain.rms_norm(tensors["embed"][special], tensors["l0.norm1"], 1e-5)
    key_dir = tensors["l0.mix.k"] @ h                              # one kv head: [dim]
    key_dir[:rot] = 0.0                                            # (the rotated pairs lie in the first `rot` features)
    key_dir /= key_dir.norm()
    for head in range(2):                                          # the alignment with u sets every query along key_dir
        tensors["l0.mix.q"][head * dimq:(head + 1) * dimq] += 6.0 * torch.outer(key_dir, u)
    tensors["l0.mix.q.norm"][:] = 3.0                              # long queries: a sharp softmax
    folder = os.path.join(str(model_root), f"sofudra_standout_{dtype}")
    write_model(folder, WINDOWED, {n: t.to(stored(dtype)) for n, t in tensors.items()})
    return folder, special


@pytest.mark.parametrize("where", ["prompt", "decoded"])
def test_one_key_inside_and_outside_a_window(model_root, where):
    """One token id occurs once, at position 40, and every later query of the first layer scores its key far above all
    others for as long as it is in the window of 21.  The logits where that key is the window's oldest one and where it
    has just left it are compared with the oracle, as rows of a prompt's portion and as single decoded tokens; the
    windows (21 and 64) lie across pages of 16."""
    dtype = "float32"
    folder, special = standout_model(model_root, dtype)
    vocab = WINDOWED["vocab"]
    ids = [t if t != special else special + 1 for t in seeded_ids(120, vocab, 31)]
    ids[40] = special
    want = plain_logits(folder, ids)
    eng = engine_for(folder, dtype, 128, 16, kv_split=64)
    edge = 40 + 21                       # the first position whose window (21) no longer holds position 40
    if where == "prompt":
        steps = [{"entries": [{"id": "x", "tokens": ids[:50], "want": list(range(50))}]},
                 {"entries": [{"id": "x", "tokens": ids[50:], "want": list(range(70))}], "end": ["x"]}]
    else:
        steps = [{"entries": [{"id": "x", "tokens": ids[:45], "want": list(range(45))}]}]
        steps += [{"entries": [{"id": "x", "tokens": [ids[i]], "want": [0]}]} for i in range(45, 120)]
    got = rl.run_in_process(eng, steps)
    check_against_plain(got, folder, {"x": ids}, 10 * TOL_F32)
    # the stand-out key matters: with a window one position longer or shorter the rows at the edge are others
    cfg, w = plain.read_folder(folder, torch.float64)
    for size, at in ((22, edge), (20, edge - 1)):
        other = json.loads(json.dumps(cfg))
        other["layers"][0]["mixer"]["mask"]["size"] = size
        moved = rel_err(plain.forward(other, w, ids)[at], want[at])
        assert moved > 1e-2, (size, moved)


def test_a_sink_that_carries_the_softmax(model_root):
    """Sinks far above the scores (the heads then give almost nothing) and far below them (an ordinary softmax), head
    by head: the engine follows the oracle, and leaving the sinks out would change the logits altogether."""
    folder = make_model(model_root, "odd", seed=7, dtype=torch.float32)
    cfg, w = plain.read_folder(folder, torch.float64)
    tensors = {n: t.clone() for n, t in w.items()}
    for name in [n for n in tensors if n.endswith(".sink")]:
        tensors[name] = torch.tensor([6.0, -30.0, 2.0, 0.0, 9.0, -4.0], dtype=torch.float64)[:tensors[name].numel()]
    folder2 = os.path.join(str(model_root), "sofudra_sinks")
    write_model(folder2, cfg, {n: t.float() for n, t in tensors.items()})
    ids = seeded_ids(90, cfg["vocab"], 4)
    eng = engine_for(folder2, "float32", 128, 8)
    steps = [{"entries": [{"id": "x", "tokens": ids[:61], "want": list(range(61))}]}]
    steps += [{"entries": [{"id": "x", "tokens": [ids[i]], "want": [0]}]} for i in range(61, 90)]
    got = rl.run_in_process(eng, steps)
    check_against_plain(got, folder2, {"x": ids}, TOL_F32)
    none = {n: (t - 100.0 if n.endswith(".sink") else t) for n, t in tensors.items()}
    assert rel_err(plain.forward(cfg, none, ids), plain_logits(folder2, ids)) > 1e-2


def test_long_decoding(model_root):
    """A short prompt, then 280 tokens one by one across page, split, chunk and window borders, beside a second request
    that decodes too; in float32 against the plain logits."""
    folder = make_model(model_root, "odd", seed=11, dtype=torch.float32)
    vocab = CONFIGS["odd"][0]["vocab"]
    a, b = seeded_ids(290, vocab, 21), seeded_ids(200, vocab, 22)
    eng = engine_for(folder, "float32", 576, 16, kv_split=64)
    steps = [{"entries": [{"id": "a", "tokens": a[:10], "want": [9]}, {"id": "b", "tokens": b[:3], "want": [2]}]}]
    for i in range(10, 290):
        ents = [{"id": "a", "tokens": [a[i]], "want": [0]}]
        j = i - 7
        if j < 200:
            ents.append({"id": "b", "tokens": [b[j]], "want": [0]})
        steps.append({"entries": ents, "end": []})
    got = rl.run_in_process(eng, steps)
    wa, wb = plain_logits(folder, a), plain_logits(folder, b)
    for (rid, p), row in got.items():
        want = (wa if rid == "a" else wb)[p]
        assert rel_err(row, want) < TOL_F32, (rid, p)


@pytest.mark.parametrize("cut", [2, 6, 7, 8, 13, 14, 15, 16, 17, 39, 40, 41, 63, 64, 65, 79, 80, 128, 129, 255, 256, 257])
def test_portion_borders(model_root, cut):
    """A prompt cut just before, at and just behind the borders of the windows (7, 13, 40), the pages (8), the
    attention's tiles (64) and splits (256), the chunks of the state's sums (64) and the number of rows from which a
    portion runs in chunks (16): the second portion's first tokens reach back over the border."""
    folder = make_model(model_root, "odd", seed=5, dtype=torch.float32)
    ids = seeded_ids(cut + 25, CONFIGS["odd"][0]["vocab"], cut)
    eng = engine_for(folder, "float32", 320, 8, kv_split=256)
    steps = [{"entries": [{"id": "x", "tokens": ids[:cut], "want": [cut - 2, cut - 1]}]},
             {"entries": [{"id": "x", "tokens": ids[cut:cut + 3], "want": [0, 1, 2]}]},
             {"entries": [{"id": "x", "tokens": ids[cut + 3:cut + 4], "want": [0]}]},
             {"entries": [{"id": "x", "tokens": ids[cut + 4:], "want": list(range(21))}], "end": ["x"]}]
    got = rl.run_in_process(eng, steps)
    want = plain_logits(folder, ids)
    for (rid, p), row in got.items():
        assert rel_err(row, want[p]) < TOL_F32, p


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_slots_and_pages_used_again(model_root, dtype):
    """Two request slots and a pool of four pages for six requests that come and go: every request must come out as
    if it ran alone, whatever its pages and its state's slot held before."""
    folder = make_model(model_root, "odd", seed=2, dtype=stored(dtype))
    vocab = CONFIGS["odd"][0]["vocab"]
    reqs = {f"q{i}": seeded_ids(n, vocab, 40 + i) for i, n in enumerate([20, 31, 12, 26, 17, 30])}
    eng = engine_for(folder, dtype, 64, 16, max_requests=2)
    names = list(reqs)
    steps = []
    for k in range(0, 6, 2):
        a, b = names[k], names[k + 1]
        ia, ib = reqs[a], reqs[b]
        steps.append({"entries": [{"id": a, "tokens": ia[:7], "want": list(range(7))}]})
        steps.append({"entries": [{"id": a, "tokens": ia[7:9], "want": [0, 1]}, {"id": b, "tokens": ib[:5], "want": list(range(5))}]})
        steps.append({"entries": [{"id": b, "tokens": ib[5:], "want": list(range(len(ib) - 5))},
                                  {"id": a, "tokens": ia[9:], "want": list(range(len(ia) - 9))}], "end": [a, b]})
    got = rl.run_in_process(eng, steps)
    eng.cache.check()
    check_against_plain(got, folder, reqs, TOL_F32 if dtype == "float32" else TOL_BF16)


def test_a_window_gives_its_pages_back(model_root):
    """All layers of this model have windows (21 and 64 positions): a request of 200 positions on a pool of 8 pages of
    16 runs through, because pages wholly behind every window are handed back; the logits are the oracle's."""
    folder = make_model(model_root, "windowed", seed=5, dtype=torch.float32, config_json=WINDOWED)
    ids = seeded_ids(200, WINDOWED["vocab"], 3)
    eng = engine_for(folder, "float32", 128, 16, max_context=256)
    steps = [{"entries": [{"id": "x", "tokens": ids[:30], "want": list(range(30))}]}]
    steps += [{"entries": [{"id": "x", "tokens": ids[i:i + 17], "want": list(range(len(ids[i:i + 17])))}]} for i in range(30, 200, 17)]
    got = rl.run_in_process(eng, steps)
    assert eng.cache.pages_held("x") <= 6
    check_against_plain(got, folder, {"x": ids}, TOL_F32)


@pytest.mark.parametrize("name,dtype", [("odd", "float32"), ("even", "bfloat16"), ("even", "float32"), ("sharp", "float32")])
def test_decoding_as_a_replayed_graph(model_root, name, dtype):
    """Engine.decode (the decoding step captured once per batch size and replayed) against the plain logits of the
    tokens it was fed, for three requests of unequal lengths, one of which ends early so that a padded row runs beside
    the others; the states of the passes of a loop advance inside the graph."""
    folder = make_model(model_root, name, seed=11, dtype=stored(dtype))
    vocab = CONFIGS[name][0]["vocab"]
    seqs = {"a": seeded_ids(40, vocab, 1), "b": seeded_ids(23, vocab, 2), "c": seeded_ids(31, vocab, 3)}
    heads = {"a": 17, "b": 3, "c": 9}
    eng = engine_for(folder, dtype, 256, CONFIGS[name][1], use_graphs=True)
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    eng.step([(r, seqs[r][:heads[r]], []) for r in seqs])
    at = dict(heads)
    live = ["a", "b", "c"]
    while live:
        eng.decode(live, [seqs[r][at[r]] for r in live])
        logits = eng.decode_graph(len(live)).logits
        for i, r in enumerate(live):
            want = plain_logits(folder, seqs[r])[at[r]]
            assert rel_err(logits[i], want) < tol, (r, at[r])
            at[r] += 1
        for r in [r for r in live if at[r] == len(seqs[r])]:
            eng.release(r)
            live.remove(r)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(model_root, dtype):
    """Engine.generate (scheduler, portions under a budget, decoding graphs, sampler) for prompts of unequal length
    on fewer slots than prompts: every generated token is the plain implementation's choice wherever that choice is
    clear, teacher-forced on the engine's own tokens."""
    folder = make_model(model_root, "odd", seed=11, dtype=stored(dtype))
    vocab = CONFIGS["odd"][0]["vocab"]
    prompts = [seeded_ids(n, vocab, 60 + n) for n in (5, 37, 18, 64, 2)]
    from beglin_b200 import Engine
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=512, page_size=16, max_requests=3)
    outs = eng.generate(prompts, max_new_tokens=12, stop_ids=(), max_step_tokens=24)
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    pinned = 0
    for prompt, out in zip(prompts, outs):
        assert len(out) == 12
        logits = plain_logits(folder, list(prompt) + list(out))
        for k, tok in enumerate(out):
            row = logits[len(prompt) + k - 1]
            top = torch.topk(row, 2).values
            slack = 2 * tol * float(row.abs().max())
            assert float(top[0] - row[tok]) <= slack, (k, tok)
            if float(top[0] - top[1]) > slack:
                assert tok == int(row.argmax()), (k, tok)
                pinned += 1
    assert pinned >= 30
    one = eng.generate([prompts[1]], max_new_tokens=12, stop_ids=())       # alone: the same tokens as in the batch
    if dtype == "float32":
        assert one[0] == outs[1]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_root, tmp_path, dtype):
    """bin/trace_run as a user runs it: JSON lines in, <step>.f32 files out, `done <step>` after each."""
    folder = make_model(model_root, "odd", seed=11, dtype=stored(dtype))
    reqs = {k: v for k, v in list(requests_for("odd").items())[:5]}
    steps, peak = rl.mixed(reqs, seed=8)
    steps = rl.number(steps)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    cmd = [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
           "--out", str(out), "--max-tokens", str(peak)]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    r = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    vocab = CONFIGS["odd"][0]["vocab"]
    got, held = {}, {}
    for s in steps:
        n_want = sum(len(e["want"]) for e in s["entries"])
        path = out / f"{s['step']}.f32"
        if n_want == 0:
            assert not path.exists()
            continue
        arr = np.fromfile(path, dtype="<f4").reshape(n_want, vocab)
        row = 0
        for e in s["entries"]:
            start = held.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], start + w)] = torch.from_numpy(arr[row].copy())
                row += 1
            held[e["id"]] = start + len(e["tokens"])
    check_against_plain(got, folder, reqs, TOL_F32 if dtype == "float32" else TOL_BF16)


def test_command_line_greedy(model_root, tmp_path):
    """`qwen_infer greedy N` on a Sofudra folder: the registry picks the architecture from config.json, and the
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
