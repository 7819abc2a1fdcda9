#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen2.5-1.5B layer sizes, random weights, bf16.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 4096] [--layers N] [--sizes 1.5b]
    python bench.py --impl reference ...      # prints the reference arm's `unavailable` line

A step is one decoding step of `batch` requests, each holding close to `context` positions in the
paged cache.  It prints ONE JSON line: `value` is decoded tokens a second on the device (the step
replayed as a CUDA graph, sampled tokens fed back on the device); `e2e` is the same through the
Python entry point `Engine.decode`, host token ids in from pinned memory and sampled ids read back
every step; `prefill` is one 2,048-token prompt in one step; `roofline` sets the bytes a decoding
step has to read (every weight once and the cache of the live requests) against the measured copy
bandwidth; `points` holds decoding at batch 1 and 64, and the other configurations of the baseline
record, each with its own engine, built and freed in turn: `decode_b8_page16` (the headline sizes with
pages of 16 positions), `gen_7b_*` (Qwen2.5-7B sizes, context 8192: 32 requests with seeded prompt lengths
of 128 to 2,048 tokens and 256 new tokens each through `Engine.generate`) and `decode_14b_b64` (Qwen2.5-14B
sizes, 64 prompts of 4,096 tokens, context limit 16384), the decoding points with milliseconds per step and
their fraction of the copy bandwidth.  `--no-big` leaves the 7B and 14B points out.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Qwen2.5-1.5B layer sizes: the third configuration of the baseline record.
CONFIG_1P5B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 28, "hidden_size": 1536, "num_attention_heads": 12, "num_key_value_heads": 2,
    "intermediate_size": 8960, "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "use_sliding_window": False, "hidden_act": "silu",
    "max_position_embeddings": 32768,
}
# Other layer sizes of the same architecture, for measurements beside the default one (--sizes).
_BIG = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "rope_theta": 1000000.0, "use_sliding_window": False,
        "hidden_act": "silu", "max_position_embeddings": 32768, "tie_word_embeddings": False, "vocab_size": 152064}
SIZES = {
    "1.5b": ("Qwen2.5-1.5B", CONFIG_1P5B),
    "0.5b": ("Qwen2.5-0.5B", dict(CONFIG_1P5B, num_hidden_layers=24, hidden_size=896, num_attention_heads=14,
                                  intermediate_size=4864)),
    "7b": ("Qwen2.5-7B", dict(_BIG, num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
                              intermediate_size=18944, rms_norm_eps=1e-6)),
    "14b": ("Qwen2.5-14B", dict(_BIG, num_hidden_layers=48, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                                intermediate_size=13824, rms_norm_eps=1e-5)),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        out = {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
        if "bf16_tflops_sustained" in p:
            out["bf16_tflops_sustained"] = float(p["bf16_tflops_sustained"])
        return out
    except (OSError, KeyError, ValueError, TypeError):
        return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.samples, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower() == "active" for s in self.samples)]
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


def kv_bytes_per_token(cfg, layers):
    hd = cfg["hidden_size"] // cfg["num_attention_heads"]
    return layers * 2 * cfg["num_key_value_heads"] * hd * 2


def prefill_flops(cfg, layers, T):
    d, im, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    hd = d // cfg["num_attention_heads"]
    qd, kvd = cfg["num_attention_heads"] * hd, cfg["num_key_value_heads"] * hd
    linear = 2.0 * T * layers * (d * (qd + 2 * kvd) + qd * d + 3 * d * im)
    attn = layers * 4.0 * qd * (T * (T + 1) / 2.0)
    head = 2.0 * d * V                     # the last row only
    return linear + attn + head


def fill_cache(eng, rids, length, seed, chunk=2048):
    """Prefill every request to `length` positions with seeded uniform token ids, through the step
    function, a few requests at a time."""
    import torch
    g = torch.Generator().manual_seed(seed)
    per_step = max(1, 8192 // min(length, chunk))
    for lo in range(0, len(rids), per_step):
        group = rids[lo:lo + per_step]
        ids = {r: torch.randint(0, eng.vocab, (length,), generator=g).tolist() for r in group}
        for p in range(0, length, chunk):
            eng.step([(r, ids[r][p:p + chunk], []) for r in group], check=False)
    torch.cuda.synchronize()


def time_decode(eng, batch, context, steps, warmup, seed, e2e, start_len=None):
    """(ms per step on the device, launches of this package's kernels in the timed region).  With
    `e2e` every step takes its tokens from the host and reads the sampled ones back.  The requests hold
    `start_len` positions before the first step (default: so that the last timed step ends at `context`)."""
    import torch
    from beglin_b200.csrc import ops
    rids = [("bench", batch, i) for i in range(batch)]
    if start_len is None:
        start_len = context - (warmup + steps) - 1
    fill_cache(eng, rids, start_len, seed)
    g = torch.Generator().manual_seed(seed + 1)
    toks = torch.randint(0, eng.vocab, (batch,), generator=g).tolist()
    if e2e:
        for _ in range(warmup):
            toks = eng.decode(rids, toks, read_back=True)
    else:
        eng.decode(rids, toks, read_back=False)          # host tokens once; then fed back on the device
        for _ in range(warmup - 1):
            eng.decode(rids, None, read_back=False)
    torch.cuda.synchronize()
    before = ops.launch_count()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    h2d = 0
    if e2e:
        for _ in range(steps):
            toks = eng.decode(rids, toks, read_back=True)
            h2d += eng.decode_graph(batch).h2d_bytes
    else:
        for _ in range(steps):
            eng.decode(rids, None, read_back=False)
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / steps
    launches = ops.launch_count() - before
    ops.raise_on_status(eng.ctx.status)
    for r in rids:
        eng.release(r)
    return ms, launches, h2d / steps


def decode_timeline(eng, batch, context, seed):
    """The kernels of ONE decode step as the device ran them (CUPTI records through torch.profiler): for
    every kernel its start and end relative to the step's first kernel, in microseconds.  Under
    programmatic dependent launch a kernel starts while the one before it still runs and then waits, so
    what a kernel adds to the step is the difference between its end and the end of the kernel before."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    rids = [("timeline", batch, i) for i in range(batch)]
    fill_cache(eng, rids, context - 16, seed)
    toks = torch.randint(0, eng.vocab, (batch,), generator=torch.Generator().manual_seed(seed)).tolist()
    eng.decode(rids, toks, read_back=False)
    for _ in range(4):
        eng.decode(rids, None, read_back=False)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(2):
            eng.decode(rids, None, read_back=False)
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA
          and "memcpy" not in e.name.lower() and "memset" not in e.name.lower()]
    ev.sort(key=lambda e: e.time_range.start)
    first = [i for i, e in enumerate(ev) if "embed_gather" in e.name][-1]
    step = ev[first:]
    t0 = step[0].time_range.start
    for r in rids:
        eng.release(r)

    def short(name):
        return name.replace("void bg::", "").replace("bg::", "").split("<")[0].split("(")[0]
    return [(short(e.name), e.time_range.start - t0, e.time_range.end - t0) for e in step]


def print_timeline(rows, layers):
    print(f"{len(rows)} kernels, {rows[-1][2]:.1f} us from the first kernel's start to the last one's end")
    print("  #  kernel                               start      end   adds")
    prev = 0.0
    shown = list(range(min(len(rows), 24))) + list(range(max(24, len(rows) - 6), len(rows)))
    for i, (name, s, e) in enumerate(rows):
        if i in shown:
            print(f"{i:4d} {name[:34]:34s} {s:8.1f} {e:8.1f} {e - prev:6.1f}")
        elif i == 24:
            print("     ...")
        prev = max(prev, e)
    adds, prev = {}, 0.0
    for name, s, e in rows:
        a = adds.setdefault(name, [0, 0.0])
        a[0] += 1
        a[1] += max(0.0, e - prev)
        prev = max(prev, e)
    print("what each kind of kernel adds to the step (its end minus the end of the kernel before it):")
    for name, (n, t) in sorted(adds.items(), key=lambda kv: -kv[1][1]):
        print(f"  {name[:40]:40s} x{n:<4d} {t:8.1f} us  ({t / n:5.1f} us each)")


def prefill_timeline(eng, T, seed):
    """The kernels of ONE prompt step of T tokens as the device ran them: (name, start, end) in microseconds
    from the step's first kernel, library kernels included."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, eng.vocab, (T,), generator=g).tolist()
    for _ in range(3):
        eng.step([("timeline", ids, [T - 1])], end=["timeline"], check=False)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        eng.step([("timeline", ids, [T - 1])], end=["timeline"], check=False)
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA
          and "memcpy" not in e.name.lower() and "memset" not in e.name.lower()]
    ev.sort(key=lambda e: e.time_range.start)
    t0 = ev[0].time_range.start

    def short(name):
        return name.replace("void bg::", "").replace("bg::", "").split("<")[0].split("(")[0]
    return [(short(e.name), e.time_range.start - t0, e.time_range.end - t0) for e in ev]


def print_busy(rows):
    """Per kind of kernel the time it ran (not what it adds), and the time in which the device ran nothing."""
    busy, idle, prev = {}, 0.0, 0.0
    for name, s, e in rows:
        b = busy.setdefault(name, [0, 0.0])
        b[0] += 1
        b[1] += e - s
        idle += max(0.0, s - prev)
        prev = max(prev, e)
    print(f"the device ran nothing for {idle:.1f} us of the step; time each kind of kernel ran:")
    for name, (n, t) in sorted(busy.items(), key=lambda kv: -kv[1][1]):
        print(f"  {name[:40]:40s} x{n:<4d} {t:8.1f} us  ({t / n:6.1f} us each)")


def time_prefill(eng, T, reps, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    best = float("inf")
    for i in range(reps + 2):
        ids = torch.randint(0, eng.vocab, (T,), generator=g).tolist()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        eng.step([("prefill", ids, [T - 1])], end=["prefill"], check=False)
        t1.record()
        torch.cuda.synchronize()
        if i >= 2:
            best = min(best, t0.elapsed_time(t1))
    return best


def free_engine(eng):
    """Drop an engine and everything it holds on the device (its graphs refer back to it, so the cycle
    collector has to run before the memory is free)."""
    import gc
    import torch
    eng._graphs.clear()
    eng.portions.graphs.clear()
    del eng
    gc.collect()
    torch.cuda.empty_cache()


def decode_point(cfg, pk, batch, context, start_len, steps, warmup, page, max_context=None, seed=5):
    """One decoding measurement with an engine of its own: tokens a second, milliseconds a step, the bytes a
    step has to read and their fraction of the copy bandwidth."""
    from beglin_b200 import Engine
    layers = cfg["num_hidden_layers"]
    eng = Engine.random(cfg, seed=0, dtype="bfloat16", device="cuda:0", max_tokens=batch * (context + 2 * page), page_size=page,
                        max_requests=batch, max_context=max_context or context)
    weight_bytes = eng.model.weight_bytes()
    ms, _, _ = time_decode(eng, batch, context, steps, warmup, seed=seed, e2e=False, start_len=start_len)
    free_engine(eng)
    first = start_len if start_len is not None else context - (warmup + steps) - 1
    mid = first + warmup + steps / 2.0
    step_bytes = weight_bytes + batch * mid * kv_bytes_per_token(cfg, layers)
    gbs = step_bytes / (ms * 1e-3) / 1e9
    return {"tok_s": round(batch * 1000.0 / ms, 1), "ms": round(ms, 4), "gb": round(step_bytes / 1e9, 3),
            "frac": round(gbs / pk["hbm_gbs"], 4), "steps": steps}


def generate_point(cfg, requests=32, new_tokens=256, context=8192, seed=11):
    """The mixed workload of the baseline record's fourth configuration through `Engine.generate`: `requests`
    prompts of seeded lengths 128..2,048 (seeded uniform token ids), `new_tokens` new tokens each, all live at
    once, host token ids in and out.  The first run captures the graphs; the second is timed on the host's
    clock between two device synchronisations."""
    import torch
    from beglin_b200 import Engine
    g = torch.Generator().manual_seed(seed)
    lengths = torch.randint(128, 2049, (requests,), generator=g).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lengths]
    eng = Engine.random(cfg, seed=0, dtype="bfloat16", device="cuda:0", max_tokens=requests * (2048 + new_tokens + 64),
                        page_size=64, max_requests=requests, max_context=context)
    out = {}
    for timed in (False, True):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = eng.generate(prompts, max_new_tokens=new_tokens, stop_ids=(), max_batch=requests, max_step_tokens=4096)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        c = eng.last_counters
        new = sum(len(o) for o in outs)
        out = {"new_tok_s": round(new / wall, 1), "tok_s_with_prompts": round((new + sum(lengths)) / wall, 1),
               "wall_s": round(wall, 3), "prompt_tokens": sum(lengths), "new_tokens": new, "steps": c.steps,
               "mixed_steps": c.mixed_steps, "preemptions": c.preemptions,
               "tbt_max_ms": round(c.gap_max_s * 1e3, 2), "tbt_mean_ms": round(c.gap_mean_s() * 1e3, 3)}
    free_engine(eng)
    return out


# ---------------------------------------------------------------------------------------------------------------
# The Sukisun decoder beside the Qwen2 decoder at equal layer sizes (--design sukisun): layer patterns and sizes
# in the manner of real models of that kind (attention through a latent with a shared rotated key part, every
# other attention layer reading its neighbour's cache, Mamba-2 layers of twice the width between them, a dense
# feed-forward of four times the width), random weights.  The Qwen2 model beside it has the same width, number
# of layers, heads and vocabulary, and a SwiGLU feed-forward with the same number of weights (three matrices of
# 2/3 the inner size).
def sukisun_config(width, heads, layers, vocab=32768):
    lat = lambda kv_from=None: dict({"heads": heads, "dim": 64, "rot_dim": 64, "vdim": 128, "q_rank": width // 2,
                                     "kv_rank": width // 4 if width <= 2048 else 512, "scale": 128 ** -0.5,
                                     "rot": {"base": 10000.0, "dims": 64}}, **({} if kv_from is None else {"kv_from": kv_from}))
    mam = {"heads": 2 * width // 128, "vdim": 128, "state": 128, "groups": 1, "conv": 4, "norm_groups": 1}
    ff = {"kind": "dense", "ff": 4 * width}
    out = []
    for i in range(layers):
        k = i % 4
        if k == 2:
            out.append({"type": "mamba2", "mixer": mam, "mlp": None})
        else:
            out.append({"type": "latent_attention", "mixer": lat(i - 1 if k == 1 else None), "mlp": ff})
    return {"architecture": "Sukisun", "vocab": vocab, "width": width, "embedding": {"scale": float(width) ** 0.5},
            "norm": {"eps": 1e-5}, "layers": out}


def qwen2_like(width, heads, layers, vocab=32768):
    return {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": layers, "hidden_size": width,
            "num_attention_heads": heads, "num_key_value_heads": max(1, heads // 4 if heads % 4 == 0 and heads > 12 else heads // 6), "intermediate_size": (8 * width // 3) // 128 * 128,
            "vocab_size": vocab, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
            "use_sliding_window": False, "hidden_act": "silu", "max_position_embeddings": 32768}


# The Nadilorn decoder beside the Qwen2 decoder at equal layer sizes (--design nadilorn): grouped-query attention with
# keys of 128 features and values of 128 or 64, a norm over the whole query and key rows, rotation of half of every head,
# a window of 1,024 positions, the enlarged softmax denominator and the output gate; the first layer with a gated GELU
# feed-forward, the others with eight routed experts of which two are chosen (inner size such that the two chosen have
# the weights of the Qwen2 layer's feed-forward).  Random weights.
def nadilorn_config(width, heads, layers, vocab=32768, vdim=128):
    kv = max(1, heads // 4 if heads % 4 == 0 and heads > 12 else heads // 6)
    mixer = {"heads": heads, "kv_heads": kv, "dim": 128, "vdim": vdim, "scale": 128 ** -0.5, "mask": {"size": 1024},
             "rot": {"base": 1000000.0, "dims": 64, "scaling": {"factor": 4.0}}}
    im = (8 * width // 3) // 128 * 128
    dense = {"kind": "dense", "ff": im}
    moe = {"kind": "moe", "expert": {"ff": (3 * im // 4) // 64 * 64}, "router": {"experts": 8, "top": 2}}
    return {"architecture": "Nadilorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "layers": [{"type": "attention", "mixer": mixer, "mlp": dense if i == 0 else moe} for i in range(layers)]}


# The Sofudra decoder beside another design at equal layer sizes (--design sofudra): a first layer of grouped-query
# attention with heads of 128 features normed one by one, whole heads rotated with stretched frequencies, a window of
# 1,024 positions and a learned sink; then layers of two mixers side by side (attention without rotation, scores squashed
# at 50, one gate per head; beside it linear attention with a constant decay per head, width / 128 heads of 128 x 128
# values of state), every layer with a dense GELU feed-forward of the Qwen2 layer's weights (two matrices of 3/2 its inner
# size) read from the same stream as the mixer.  Two of the layers are passed twice with the input mix in front, so that
# the number of layer runs is the other model's number of layers.  Random weights.
def sofudra_config(width, heads, layers, vocab=32768):
    kv = max(1, heads // 4 if heads % 4 == 0 and heads > 12 else heads // 6)
    first = {"heads": heads, "kv_heads": kv, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": 1024},
             "rot": {"base": 1000000.0, "dims": 128, "scaling": {"factor": 4.0, "original": 4096, "fast": 16.0, "slow": 2.0}}}
    left = {"heads": heads, "kv_heads": kv, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "softcap": 50.0}
    dh = width // 128
    right = {"heads": dh, "dim": 128, "vdim": 128, "decay": [1.0 - 2.0 ** (-3.0 - 5.0 * i / max(1, dh - 1)) for i in range(dh)]}
    ff = {"kind": "dense", "ff": (4 * width) // 128 * 128}
    par = {"left": left, "right": right, "left_scale": 1.0, "right_scale": 1.0}
    k = 2 if layers >= 5 else 1                    # layers passed twice
    n = layers - k
    return {"architecture": "Sofudra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": float(width) ** 0.5},
            "residual_mult": 0.5, "logit_softcap": 30.0, "loop": {"start": 1, "stop": 1 + k, "times": 2},
            "layers": [{"type": "attention" if i == 0 else "parallel", "mixer": first if i == 0 else par, "mlp": ff} for i in range(n)]}


# The Tuzupel decoder beside another design at equal layer sizes (--design tuzupel): the residual in two lanes; layers in the
# order attention, latent attention, recurrence, attention, ...: grouped-query attention with heads of 128 features normed
# one by one, half of every head rotated in neighbouring pairs with band-scaled frequencies, blocks of 1,024 positions and a
# learned sink; attention through a latent of 512 features (width / 4 up to width 2048) with heads of 128 and a window of
# 1,024; a gated linear recurrence of the model's width in parts of 256 channels behind a convolution of 4 taps.  Every
# layer has eight routed experts with a gate branch of which two are chosen, two identity experts beside them and a shared
# expert; the chosen two and the shared one together have the weights of the Qwen2 layer's feed-forward.  Random weights.
def tuzupel_config(width, heads, layers, vocab=32768):
    kv = max(1, heads // 4 if heads % 4 == 0 and heads > 12 else heads // 6)
    att = {"heads": heads, "kv_heads": kv, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": 1024},
           "rot": {"base": 500000.0, "dims": 64, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    lat = {"heads": heads, "dim": 128, "vdim": 128, "kv_rank": width // 4 if width <= 2048 else 512, "scale": 128 ** -0.5,
           "mask": {"size": 1024}}
    rec = {"width": width, "blocks": width // 256, "conv": 4}
    im = (8 * width // 3) // 128 * 128
    moe = {"kind": "moe", "expert": {"ff": (im // 4) // 64 * 64, "limit": 7.0},
           "router": {"experts": 8, "identity": 2, "scale": 2.5, "top": 2}, "shared": {"ff": (im // 2) // 64 * 64, "limit": 7.0}}
    kinds = [("attention", att), ("latent_attention", lat), ("rglru", rec)]
    return {"architecture": "Tuzupel", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "streams": 2, "logit_softcap": 30.0,
            "layers": [{"type": kinds[i % 3][0], "mixer": kinds[i % 3][1], "mlp": moe} for i in range(layers)]}


DESIGN_SIZES = {"1536": (1536, 12, 8), "4096": (4096, 32, 4)}      # width -> (width, heads, layers)
DESIGNS = {"sukisun": lambda w, h, l: sukisun_config(w, h, l), "nadilorn": lambda w, h, l: nadilorn_config(w, h, l),
           "nadilorn-v64": lambda w, h, l: nadilorn_config(w, h, l, vdim=64), "sofudra": lambda w, h, l: sofudra_config(w, h, l),
           "tuzupel": lambda w, h, l: tuzupel_config(w, h, l)}
BESIDE = dict(DESIGNS, qwen2=lambda w, h, l: qwen2_like(w, h, l))


def phase_times(eng, fn):
    """Device milliseconds per kernel class of one call of fn (kernel by kernel, CUDA events around every class)."""
    import torch
    from beglin_b200.csrc import ops
    graphs, eng.use_graphs = eng.use_graphs, False
    fn()                                   # warm
    torch.cuda.synchronize()
    ops.profile_begin()
    fn()
    rec = ops.profile_end()
    eng.use_graphs = graphs
    return {k: round(ms, 4) for k, (ms, _) in rec.items()}


def design_point(cfg, pk, batch, context, steps, warmup, tokens):
    """Decoding (replayed graph) and one prompt step of `tokens` tokens for one configuration, with the device time per
    kernel class of the prompt step and of one decoding step run kernel by kernel."""
    import torch
    from beglin_b200 import Engine
    page = 64
    eng = Engine.random(cfg, seed=0, dtype="bfloat16", device="cuda:0", max_tokens=batch * (context + page), page_size=page,
                        max_requests=batch, max_context=context + page)
    kv_bytes = sum(g.device_pool.numel() * g.device_pool.element_size() for g in eng.cache.kv_groups if g.device_pool is not None)
    state_bytes = eng.cache.device_bytes() - kv_bytes      # per-request state of fixed size: read and written every step
    out = {"weight_gb": round(eng.model.weight_bytes() / 1e9, 3), "cache_bytes_per_token": kv_bytes // max(1, eng.cache.num_pages + 1) // page,
           "state_bytes_per_request": state_bytes // max(1, batch)}
    pms = time_prefill(eng, tokens, reps=3, seed=3)
    out["prefill_tok_s"] = round(tokens * 1000.0 / pms, 1)
    out["prefill_ms"] = round(pms, 3)
    g = torch.Generator().manual_seed(9)
    ids = torch.randint(0, eng.vocab, (tokens,), generator=g).tolist()
    out["prefill_classes_ms"] = phase_times(eng, lambda: eng.step([("p", ids, [tokens - 1])], end=["p"], check=False))
    ms, launches, _ = time_decode(eng, batch, context, steps, warmup, seed=1, e2e=False)
    out["decode_tok_s"] = round(batch * 1000.0 / ms, 1)
    out["decode_ms"] = round(ms, 4)
    out["decode_launches_per_step"] = launches // max(1, steps)
    # (a layer with a window reads no more of a request's positions than the window holds)
    windows = [l["mixer"].get("mask", {}).get("size") for l in cfg.get("layers", []) if isinstance(l.get("mixer"), dict)]
    seen = min([context - steps / 2.0] + [w for w in windows if w]) if windows and all(windows) else context - steps / 2.0
    step_bytes = eng.model.weight_bytes() + batch * seen * out["cache_bytes_per_token"] + 2 * state_bytes
    out["decode_frac_of_hbm"] = round(step_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
    rids = [("cls", i) for i in range(batch)]
    fill_cache(eng, rids, context - 8, seed=4)
    toks = [1] * batch
    out["decode_classes_ms"] = phase_times(eng, lambda: eng.step([(r, [t], [0]) for r, t in zip(rids, toks)], check=False))
    free_engine(eng)
    return out


def design_timeline(args):
    """The kernels of one decoding step (or of one prompt step of 2,048 tokens) of the design at the first of the sizes."""
    from beglin_b200 import Engine
    width, heads, layers = DESIGN_SIZES[args.design_sizes.split(",")[0]]
    eng = Engine.random(DESIGNS[args.design](width, heads, layers), seed=0, dtype="bfloat16", device="cuda:0",
                        max_tokens=args.batch * (args.context + 64), page_size=64, max_requests=args.batch,
                        max_context=args.context + 64)
    if args.timeline == "prefill":
        rows = prefill_timeline(eng, 2048, seed=3)
        print_timeline(rows, layers)
        print_busy(rows)
    else:
        print_timeline(decode_timeline(eng, args.batch, args.context, seed=1), layers)
    return 0


def design_comparison(args, pk):
    if args.timeline:
        return design_timeline(args)
    clocks = ClockSampler()
    clocks.start()
    rows = {}
    for name in args.design_sizes.split(","):
        width, heads, layers = DESIGN_SIZES[name]
        for label, cfg in [(args.design, DESIGNS[args.design](width, heads, layers))] + \
                          [(b, BESIDE[b](width, heads, layers)) for b in args.beside.split(",") if b]:
            rows[f"{label}_{name}"] = design_point(cfg, pk, args.batch, args.context, min(args.steps, 32), args.warmup, 2048)
    print(json.dumps({"design": f"{args.design} beside {args.beside} at equal layer sizes", "dtype": "bf16", "batch": args.batch,
                      "context": args.context, "data": "synthetic (seeded uniform token ids, random weights)",
                      "peaks": pk, "clocks": clocks.stop(), "points": rows}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--sizes", default="1.5b", choices=sorted(SIZES), help="layer sizes (default: the baseline record's)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (default: all)")
    ap.add_argument("--no-points", action="store_true", help="skip decoding at batch 1 and 64 and the prefill")
    ap.add_argument("--no-big", action="store_true", help="skip the points with engines of their own (page 16, 7B, 14B)")
    ap.add_argument("--gemm", default="auto")
    ap.add_argument("--no-fuse", action="store_true", help="norms, residual adds and SwiGLU as kernels of their own")
    ap.add_argument("--timeline", nargs="?", const="decode", default=None, choices=["decode", "prefill"],
                    help="instead of the measurement: print the kernels of one decode step (or of one prompt step of "
                         "2,048 tokens) with their device times")
    ap.add_argument("--design", default=None, choices=sorted(DESIGNS),
                    help="instead of the headline measurement: this design beside Qwen2 at equal layer sizes, prefill and "
                         "decode, with the device time per kernel class")
    ap.add_argument("--beside", default="qwen2", help="what --design is measured beside: a list of " + ",".join(sorted(BESIDE)))
    ap.add_argument("--design-sizes", default="1536,4096", help="widths to compare at, of " + ",".join(sorted(DESIGN_SIZES)))
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a C program for Apple CPUs (Accelerate, NEON, SME2) with no Python "
                          "package: pip reports \"Neither 'setup.py' nor 'pyproject.toml' found\", and "
                          "qwen_infer.c does not compile on x86 Linux"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(3, args.warmup)
    if args.steps + args.warmup + 2 > args.context:          # every timed step decodes one more position
        args.context = args.steps + args.warmup + 64

    import torch
    from beglin_b200 import Engine
    pk = peaks()
    if args.design:
        return design_comparison(args, pk)
    model_name, full = SIZES[args.sizes]
    args.layers = args.layers or full["num_hidden_layers"]
    cfg = dict(full, num_hidden_layers=args.layers)
    max_batch = args.batch if args.no_points else max(args.batch, 64)
    page = 64
    eng = Engine.random(cfg, seed=0, dtype="bfloat16", device="cuda:0", max_tokens=max_batch * args.context,
                        page_size=page, max_requests=max_batch, max_context=args.context, gemm=args.gemm, fuse=not args.no_fuse)
    if args.timeline == "prefill":
        rows = prefill_timeline(eng, 2048, seed=3)
        print_timeline(rows, args.layers)
        print_busy(rows)
        return 0
    if args.timeline:
        print_timeline(decode_timeline(eng, args.batch, args.context, seed=1), args.layers)
        return 0
    weight_bytes = eng.model.weight_bytes()
    kvb = kv_bytes_per_token(cfg, args.layers)

    clocks = ClockSampler()
    clocks.start()
    ms, launches, _ = time_decode(eng, args.batch, args.context, args.steps, args.warmup, seed=1, e2e=False)
    clock_rec = clocks.stop()
    ms_e2e, _, h2d = time_decode(eng, args.batch, args.context, args.steps, args.warmup, seed=1, e2e=True)

    value = args.batch * 1000.0 / ms
    ctx_mid = args.context - 1 - args.steps / 2.0
    step_bytes = weight_bytes + args.batch * ctx_mid * kvb
    achieved = step_bytes / (ms * 1e-3) / 1e9
    out = {
        "metric": f"decode tok/s @ batch {args.batch}; {model_name} bf16", "value": round(value, 1), "unit": "tok/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (seeded uniform token ids, random weights)",
        "config": {"model": f"{model_name} sizes", "layers": args.layers, "layers_of_config": full["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["hidden_size"] // cfg["num_attention_heads"], "intermediate": cfg["intermediate_size"],
                   "vocab": cfg["vocab_size"], "tied_head": bool(cfg["tie_word_embeddings"]), "global_batch": args.batch, "seq_len": args.context,
                   "page_size": page, "parallelism": "single GPU", "weights": "random, seeded",
                   "l2": "inputs larger than L2 (weights and cache read once per step)",
                   "peaks": pk["source"]},
        "e2e": {"value": round(args.batch * 1000.0 / ms_e2e, 1), "unit": "tok/s",
                "h2d_bytes_per_step": round(h2d, 1),
                "d2h_bytes_per_step": int(args.batch * 4)},
        "gpu_launches": int(launches),
        "clocks": clock_rec,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if not args.no_points:
        points = {}
        for b in (1, 64):
            m, _, _ = time_decode(eng, b, args.context, min(args.steps, 32), args.warmup, seed=2, e2e=False)
            points[f"decode_b{b}"] = round(b * 1000.0 / m, 1)
        out["points"] = points
        T = 2048
        pms = time_prefill(eng, T, reps=3, seed=3)
        flops = prefill_flops(cfg, args.layers, T)
        out["prefill"] = {"value": round(T * 1000.0 / pms, 1), "tokens": T, "ms": round(pms, 3),
                          "frac": round(flops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        if not args.no_big and args.sizes == "1.5b" and args.layers == full["num_hidden_layers"]:
            free_engine(eng)
            del eng
            # the headline sizes with the page size the baseline record states
            p16 = decode_point(cfg, pk, args.batch, args.context, None, min(args.steps, 32), args.warmup, page=16)
            points.update({"decode_b8_page16": p16["tok_s"], "decode_b8_page16_ms": p16["ms"], "decode_b8_page16_frac": p16["frac"]})
            # Qwen2.5-7B sizes: the mixed workload through Engine.generate
            gen = generate_point(SIZES["7b"][1])
            points.update({"gen_7b_" + k: v for k, v in gen.items()})
            # Qwen2.5-14B sizes: 64 prompts of 4,096 tokens under a context limit of 16384
            big = decode_point(SIZES["14b"][1], pk, 64, 4096 + 64, 4096, 8, 3, page=64, max_context=16384)
            points.update({"decode_14b_b64": big["tok_s"], "decode_14b_b64_ms": big["ms"], "decode_14b_b64_gb": big["gb"],
                           "decode_14b_b64_frac": big["frac"], "decode_14b_b64_steps": big["steps"]})
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
