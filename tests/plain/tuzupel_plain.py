"""Plain, slow implementation of the Tuzupel decoder, used only as the oracle of the tests.

Whole sequences, no cache, one function per mechanism, float64 tensor arithmetic on the CPU.  It shares no code with the
`beglin_b200` package: the model folder is read with the `json` module and the `safetensors` library, attention is
computed query by query over explicit lists of visible keys, the recurrence token by token and the experts token by
token, so that a fault of the engine's loader, cache, batching or kernels cannot be mirrored here.

The design in this file's notation.  A model keeps n lanes L_1 .. L_n of the residual, all equal to the embedded row at
the start.  A sublayer F with norm N and lane constants (r [n], M [n, n], w [n]) reads z = sum_a r_a L_a, computes
y = F(N(z)) and replaces all lanes at once: L_b <- sum_a M[a, b] L_a + w_b y.  A layer is a mixer sublayer, then (if it has
one) a feed-forward sublayer.  N(z) = z / sqrt(mean(z^2) + eps) (1 + g).  The logits are the head's product of the final
norm of sum_a L_a, squashed by c tanh(l / c).  A model without lanes keeps one residual x <- x + F(N(x)).

Mixers: "attention" (grouped-query attention, queries and keys normed head by head with a plain weight, the leading
features of every head turned in neighbouring pairs by position with frequencies rescaled band by band, a query seeing
the earlier keys of its own block of positions only, a learned number per head in the softmax's denominator);
"latent_attention" (keys and values made from one normed low-rank row per position, a sliding window, no positions);
"rglru" (a gated linear recurrence per channel behind a short causal convolution, beside a GELU branch).

Feed-forward: routed experts with a clamped gated activation, a softmax router with a choice bias, identity experts, and
a shared expert behind a sigmoid gate of one number per token.
"""
from __future__ import annotations

import json
import math
import os
from typing import Callable, Dict, List, Optional, Sequence

import torch


def read_folder(folder: str, dtype: torch.dtype = torch.float64):
    from safetensors import safe_open

    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    weights: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(dtype)
    return cfg, weights


# ----------------------------------------------------------------------------- small functions
def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_plain(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * w


def norm_one_plus(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * (1.0 + g)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def squash(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


# ----------------------------------------------------------------------------- positions
def banded_frequencies(base: float, dims: int, scaling: Optional[dict]) -> List[float]:
    """Pair i turns at f_i = base^(-2i/dims).  With `scaling` {factor, low, high, original}: a pair whose wavelength
    2 pi / f is shorter than original/high keeps f; one longer than original/low turns at f / factor; between the two
    the blend t f + (1 - t) f / factor with t = (original / wavelength - low) / (high - low)."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"])
            original = float(scaling["original"])
            wavelength = 2.0 * math.pi / f
            if wavelength > original / low:
                f = f / factor
            elif not wavelength < original / high:
                t = (original / wavelength - low) / (high - low)
                f = (1.0 - t) * f / factor + t * f
        out.append(f)
    return out


def turn_pairs(v: torch.Tensor, positions: Sequence[int], base: float, dims: int, scaling: Optional[dict]) -> torch.Tensor:
    """v [T, heads, n]: of every head the first `dims` features turn, feature 2i together with feature 2i + 1."""
    out = v.clone()
    freqs = banded_frequencies(base, dims, scaling)
    pos = torch.tensor(list(positions), dtype=torch.float64)
    for i, f in enumerate(freqs):
        a = pos * f
        c, s = torch.cos(a).to(v.dtype)[:, None], torch.sin(a).to(v.dtype)[:, None]
        u, w = v[:, :, 2 * i], v[:, :, 2 * i + 1]
        out[:, :, 2 * i] = u * c - w * s
        out[:, :, 2 * i + 1] = w * c + u * s
    return out


# ----------------------------------------------------------------------------- attention, query by query
def visible(t: int, block: Optional[int] = None, window: Optional[int] = None) -> range:
    """The keys that query t sees: with `block` those of its own block of positions up to itself, with `window` itself
    and the window - 1 before it, else all up to itself."""
    first = 0
    if block is not None:
        first = max(first, (t // block) * block)
    if window is not None:
        first = max(first, t - window + 1)
    return range(first, t + 1)


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, see: Callable[[int], range],
                      sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, H, n], k [T, G, n], v [T, G, nv] -> [T, H, nv].  Query head h reads kv head h // (H / G).  `see(t)` lists
    the keys of query t.  `sink` [H]: exp(sink_h) joins the denominator and nothing else."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=q.dtype)
    for t in range(T):
        keys = list(see(t))
        for h in range(H):
            g = h // (H // G)
            s = (k[keys, g] @ q[t, h]) * scale
            m = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            den = e.sum() if sink is None else e.sum() + torch.exp(sink[h] - m)
            out[t, h] = (e / den) @ v[keys, g]
    return out


def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, positions: Sequence[int]) -> torch.Tensor:
    T = h.shape[0]
    H, G, n, nv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).view(T, H, n)
    k = (h @ w["k"].T).view(T, G, n)
    v = (h @ w["v"].T).view(T, G, nv)
    q, k = norm_plain(q, w["q.norm"], eps), norm_plain(k, w["k.norm"], eps)
    rot = m.get("rot")
    if rot is not None and rot["dims"]:
        q = turn_pairs(q, positions, rot["base"], rot["dims"], rot.get("scaling"))
        k = turn_pairs(k, positions, rot["base"], rot["dims"], rot.get("scaling"))
    block = m["mask"]["size"] if m.get("mask") else None
    # positions are those of the sequence itself: the rows here are a whole sequence from position 0
    o = softmax_attention(q, k, v, m["scale"], lambda t: visible(t, block=block), sink=w.get("sink"))
    return o.reshape(T, H * nv) @ w["o"].T


def latent_attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, n, nv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).view(T, H, n)
    c = norm_plain(h @ w["dkv"].T, w["dkv.norm"], eps)
    k = (c @ w["uk"].T).view(T, H, n)
    v = (c @ w["uv"].T).view(T, H, nv)
    window = m["mask"]["size"] if m.get("mask") else None
    o = softmax_attention(q, k, v, m["scale"], lambda t: visible(t, window=window))
    return o.reshape(T, H * nv) @ w["o"].T


# ----------------------------------------------------------------------------- the gated linear recurrence
def causal_taps(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, K] (the last column meets the current token), zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        acc = bias.clone()
        for j in range(K):
            src = t - (K - 1 - j)
            if src >= 0:
                acc = acc + taps[:, j] * x[src]
        out[t] = acc
    return out


def rglru_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict) -> torch.Tensor:
    T = h.shape[0]
    W, B = m["width"], m["blocks"]
    y = gelu_tanh(h @ w["y"].T + w["y.b"])
    u = causal_taps(h @ w["x"].T + w["x.b"], w["conv"], w["conv.b"])
    ub = u.view(T, B, W // B)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", w["ra"], ub) + w["ra.b"]).reshape(T, W)
    i = torch.sigmoid(torch.einsum("boi,tbi->tbo", w["ri"], ub) + w["ri.b"]).reshape(T, W)
    log_a = -8.0 * r * torch.nn.functional.softplus(w["lam"])
    a = torch.exp(log_a)
    s = torch.zeros(W, dtype=h.dtype)
    out = torch.zeros((T, W), dtype=h.dtype)
    for t in range(T):
        s = a[t] * s + torch.sqrt(1.0 - a[t] * a[t]) * (i[t] * u[t])
        out[t] = s * y[t]
    return out @ w["o"].T


# ----------------------------------------------------------------------------- feed-forward
def clamped_expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def routed_feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], f: dict) -> torch.Tensor:
    """Token by token: softmax over all router outputs, choice by score + correction, weights = scores times the
    router's scale; the last `identity` router outputs stand for experts that return their input."""
    T = h.shape[0]
    r = f["router"]
    E, I, top = r["experts"], r.get("identity", 0), r["top"]
    out = torch.zeros_like(h)
    scores = torch.softmax(h @ w["router"].T, dim=-1)
    choice = scores + w["correction"] if "correction" in w else scores
    for t in range(T):
        order = sorted(range(E + I), key=lambda e: (-float(choice[t, e]), e))[:top]
        for e in order:
            weight = scores[t, e] * r["scale"]
            if e >= E:
                out[t] = out[t] + weight * h[t]
            else:
                out[t] = out[t] + weight * clamped_expert(h[t], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"],
                                                          f["expert"]["limit"])
    if f.get("shared") is not None:
        sh = clamped_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"], f["shared"]["limit"])
        out = out + torch.sigmoid(h @ w["shared.sg"].T) * sh
    return out


# ----------------------------------------------------------------------------- the model
def sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def mixer_of(kind: str, h, w, m, eps, positions):
    if kind == "attention":
        return attention_mixer(h, w, m, eps, positions)
    if kind == "latent_attention":
        return latent_attention_mixer(h, w, m, eps)
    if kind == "rglru":
        return rglru_mixer(h, w, m)
    raise ValueError(kind)


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int], tap: Optional[Callable] = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence from position 0.  `tap(layer, rows)` gets the sum of the lanes behind
    every layer."""
    eps = cfg["norm"]["eps"]
    lanes_n = cfg.get("streams")
    x = weights["embed"][list(tokens)]
    positions = list(range(len(tokens)))
    lanes = [x.clone() for _ in range(lanes_n)] if lanes_n else None

    def sublayer(run, norm_w, hc):
        nonlocal lanes, x
        if lanes is None:
            x = x + run(norm_one_plus(x, norm_w, eps))
            return
        z = sum(hc["in"][a] * lanes[a] for a in range(lanes_n))
        y = run(norm_one_plus(z, norm_w, eps))
        lanes = [sum(hc["mix"][a, b] * lanes[a] for a in range(lanes_n)) + hc["out"][b] * y for b in range(lanes_n)]

    for li, layer in enumerate(cfg["layers"]):
        p = f"l{li}."
        w = sub(weights, p + "mix.")
        sublayer(lambda hh: mixer_of(layer["type"], hh, w, layer["mixer"], eps, positions), weights[p + "norm1"],
                 sub(weights, p + "hc1."))
        if layer.get("mlp") is not None:
            wf = sub(weights, p + "mlp.")
            sublayer(lambda hh: routed_feed_forward(hh, wf, layer["mlp"]), weights[p + "norm2"], sub(weights, p + "hc2."))
        if tap is not None:
            tap(li, sum(lanes) if lanes is not None else x)
    total = sum(lanes) if lanes is not None else x
    logits = norm_one_plus(total, weights["final.norm"], eps) @ weights["head"].T
    cap = cfg.get("logit_softcap")
    return squash(logits, cap) if cap else logits
