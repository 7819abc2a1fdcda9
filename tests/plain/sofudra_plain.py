"""Plain, slow implementation of the Sofudra decoder, used only as the oracle of the tests.

Whole sequences, no cache, one function per mechanism, float64 tensor arithmetic on the CPU.  It shares no code
with the `beglin_b200` package: the model folder is read with the `json` module and the `safetensors` library,
attention is computed query by query over explicit lists of visible keys and the recurrence token by token, so
that a fault of the engine's loader, cache, batching or kernels cannot be mirrored here.

The design in this file's notation.  e = E[token] * s_e is the embedded row.  A layer has two sublayers that read
the same stream: x <- x + m (A(N1(x)) + F(N2(x))), N an RMS norm with a weight, m one constant of the model; a
layer may lack F.  A run of consecutive layers (a loop) is passed several times with the same weights; in front of
each pass the stream is replaced by W_in [x; e].  A is one of two mixers.

"attention": grouped-query attention whose queries and keys are RMS-normed head by head (one weight vector for all
heads), then turned by position over the leading features of every head, in halves, with per-frequency stretched
angles and an amplitude on cosine and sine; a query sees itself and the w - 1 positions before it; the softmax's
denominator also holds exp(b_h), b_h a learned number of head h that belongs to no key.

"parallel": two mixers of the same input, added with two constants.  Left: grouped-query attention with biases,
normed queries and keys, no positions, scores squashed by c tanh(s / c), every earlier position visible, and every
head's result multiplied by sigmoid of one number that a further product of the input gives for it.  Right: per
head a matrix state S <- d_h S + k v^T read out as S^T q, with q, k, v = silu of three products of the input; the
joined heads are RMS-normed with a weight, multiplied by sigmoid of a fourth product, and projected.

F = W_down gelu_tanh(W_up h).  Logits: the head's product of the final norm, squashed by c tanh(l / c).
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
def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) (* w) along the last axis."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def squash(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


# ----------------------------------------------------------------------------- positions
def stretched_frequencies(base: float, dims: int, scaling: Optional[dict]):
    """(frequency of every pair, amplitude of cosine and sine).  Pair i turns at base^(-2i/dims).  With `scaling`
    {factor, original, fast, slow}: a pair whose index lies below lo keeps its frequency, one above hi has it divided
    by the factor, those between are blended linearly, where lo and hi are the indexes at which a pair completes
    `fast` and `slow` turns over `original` positions; the amplitude is 0.1 ln(factor) + 1."""
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    if scaling is None:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def index_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index_of(float(scaling["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def turn_halves(v: torch.Tensor, positions: Sequence[int], base: float, dims: int, scaling: Optional[dict]) -> torch.Tensor:
    """v [T, heads, n]: of every head the first `dims` features turn, feature i together with feature i + dims/2."""
    out = v.clone()
    half = dims // 2
    freqs, amp = stretched_frequencies(base, dims, scaling)
    pos = torch.tensor(list(positions), dtype=torch.float64)
    for i in range(half):
        a = pos * freqs[i]
        c, s = (torch.cos(a) * amp).to(v.dtype)[:, None], (torch.sin(a) * amp).to(v.dtype)[:, None]
        u, w = v[:, :, i], v[:, :, i + half]
        out[:, :, i] = u * c - w * s
        out[:, :, i + half] = w * c + u * s
    return out


# ----------------------------------------------------------------------------- attention, query by query
def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: Optional[int] = None,
                      sink: Optional[torch.Tensor] = None, cap: Optional[float] = None) -> torch.Tensor:
    """q [T, H, n], k [T, G, n], v [T, G, nv] -> [T, H, nv].  Query head h reads kv head h // (H / G).  Query t sees
    the keys j <= t, with a window only those with t - j < window.  `cap`: scores squashed.  `sink` [H]: exp(sink_h)
    joins the denominator and nothing else."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=q.dtype)
    for t in range(T):
        first = 0 if window is None else max(0, t - window + 1)
        for h in range(H):
            g = h // (H // G)
            s = (k[first:t + 1, g] @ q[t, h]) * scale
            if cap is not None:
                s = squash(s, cap)
            top = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - top)
            den = e.sum() if sink is None else e.sum() + torch.exp(sink[h] - top)
            out[t, h] = (e / den) @ v[first:t + 1, g]
    return out


def head_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x [T, heads, n]: every head's row normed by its own root mean square, times one weight vector for all heads."""
    return rms_norm(x, w, eps)


def attention_mixer(h: torch.Tensor, positions: Sequence[int], m: dict, w: Dict[str, torch.Tensor], p: str, eps: float):
    """The "attention" mixer.  h [T, width]."""
    T = h.shape[0]
    H, G, n, nv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, n)
    k = (h @ w[p + "k"].T).reshape(T, G, n)
    v = (h @ w[p + "v"].T).reshape(T, G, nv)
    q, k = head_norm(q, w[p + "q.norm"], eps), head_norm(k, w[p + "k.norm"], eps)
    rot = m.get("rot")
    if rot is not None:
        q = turn_halves(q, positions, rot["base"], rot["dims"], rot.get("scaling"))
        k = turn_halves(k, positions, rot["base"], rot["dims"], rot.get("scaling"))
    window = m["mask"]["size"] if m.get("mask") is not None else None
    o = softmax_attention(q, k, v, m["scale"], window=window, sink=w[p + "sink"])
    return o.reshape(T, H * nv) @ w[p + "o"].T


def gated_attention_mixer(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float):
    """The left half of the "parallel" mixer."""
    T = h.shape[0]
    H, G, n, nv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, n)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, n)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, nv)
    q, k = head_norm(q, w[p + "q.norm"], eps), head_norm(k, w[p + "k.norm"], eps)
    o = softmax_attention(q, k, v, m["scale"], cap=m["softcap"])
    gate = torch.sigmoid(h @ w[p + "g"].T)                      # [T, H]: one number per head
    return (o * gate[:, :, None]).reshape(T, H * nv) @ w[p + "o"].T


def decayed_state_mixer(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float,
                        state: Optional[torch.Tensor] = None):
    """The right half: S_t = d S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, head by head, from a state of nought (or
    `state` [heads, dim, vdim], which is advanced in place)."""
    T = h.shape[0]
    H, n, nv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).reshape(T, H, n)
    k = silu(h @ w[p + "k"].T).reshape(T, H, n)
    v = silu(h @ w[p + "v"].T).reshape(T, H, nv)
    S = torch.zeros((H, n, nv), dtype=h.dtype) if state is None else state
    o = torch.zeros((T, H, nv), dtype=h.dtype)
    for t in range(T):
        for a in range(H):
            S[a] = float(m["decay"][a]) * S[a] + torch.outer(k[t, a], v[t, a])
            o[t, a] = S[a].T @ q[t, a]
    y = rms_norm(o.reshape(T, H * nv), w[p + "norm"], eps) * torch.sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def parallel_mixer(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float):
    left = gated_attention_mixer(h, m["left"], w, p + "left.", eps)
    right = decayed_state_mixer(h, m["right"], w, p + "right.", eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return gelu_tanh(h @ w[p + "up"].T) @ w[p + "down"].T


# ----------------------------------------------------------------------------- the model
def run_order(cfg: dict) -> List[tuple]:
    """(layer, whether a pass of the loop begins in front of it) for every run of a layer."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if loop is None:
        return [(i, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(start)]
    for _ in range(times):
        order += [(i, i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n)]


def layer(x: torch.Tensor, positions: Sequence[int], cfg: dict, i: int, w: Dict[str, torch.Tensor]) -> torch.Tensor:
    L = cfg["layers"][i]
    eps, p = float(cfg["norm"]["eps"]), f"l{i}."
    h1 = rms_norm(x, w[p + "norm1"], eps)
    if L["type"] == "attention":
        a = attention_mixer(h1, positions, L["mixer"], w, p + "mix.", eps)
    elif L["type"] == "parallel":
        a = parallel_mixer(h1, L["mixer"], w, p + "mix.", eps)
    else:
        raise ValueError(f"layer type {L['type']}")
    if L.get("mlp") is not None:
        a = a + feed_forward(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.")
    return x + float(cfg["residual_mult"]) * a


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int],
            tap: Optional[Callable[[int, torch.Tensor], None]] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence from position 0.  `tap(run, x)` sees the stream behind every run of a
    layer."""
    positions = list(range(len(tokens)))
    e = w["embed"][torch.tensor(list(tokens), dtype=torch.long)] * float(cfg["embedding"]["scale"])
    x = e
    for run, (i, enters) in enumerate(run_order(cfg)):
        if enters:
            x = torch.cat([x, e], dim=-1) @ w["loop.in"].T
        x = layer(x, positions, cfg, i, w)
        if tap is not None:
            tap(run, x)
    logits = rms_norm(x, w["final.norm"], float(cfg["norm"]["eps"])) @ w["head"].T
    cap = cfg.get("logit_softcap")
    return squash(logits, float(cap)) if cap else logits
