"""The Sofudra decoder: its configuration, read from the keys of its own config.json, and its description as a list
of parts.

config.json names the architecture in the string `architecture`, gives `vocab`, `width`, `norm.eps`, `embedding.scale`
(the embedded rows times a constant), `residual_mult` (m below), `logit_softcap` (c tanh(logits / c)) and lists the
layers one by one: each entry gives `type` (which mixer: "attention" or "parallel"), `mixer` (its sizes and constants)
and `mlp` (`{"kind": "dense", "ff": n}`, or null for a layer without a feed-forward).  Both sublayers of a layer read
the same stream through RMS norms of their own: x <- x + m (mixer(norm1(x)) + mlp(norm2(x))).  `loop` {start, stop,
times}: the layers start .. stop-1 are passed `times` times in a row with the same weights, every pass with caches
and states of its own; in front of each pass the stream becomes W_in [x; e], e the embedded rows.  Tensors of layer i
are called `l<i>.*`.

"attention": grouped-query attention with every head of queries and keys RMS-normed by itself, rotation of the leading
`rot.dims` features in halves with frequencies stretched over a ramp (`rot.scaling` {factor, original, fast, slow}) and
an amplitude on cosine and sine, a window of `mask.size` positions and a softmax denominator that also holds exp of a
learned number per head.  "parallel": `left`, grouped-query attention with biases, normed heads, no rotation, scores
squashed at `softcap`, one sigmoid gate per head; beside `right`, linear attention with a constant decay per head;
added with `left_scale` and `right_scale`.  The feed-forward is W_down gelu_tanh(W_up h).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Iterable, List, Optional, Tuple

from ..config.reader import ConfigError, ConfigFields
from ..config.registry import Architecture, register_architecture
from ..parts.spec import (AttentionSpec, DecayAttentionSpec, DenseActSpec, EntrySpec, InputMixSpec, LayerSpec, ModelSpec,
                          NormSpec, ParallelMixersSpec, PositionSpec, Stage)


def _positive(f: ConfigFields, key: str) -> int:
    v = f.integer(key, required=True)
    if v <= 0:
        raise ConfigError(f"{f.origin}: {key}={v} must be positive")
    return v


@dataclass(frozen=True)
class StretchConfig:
    """rot.scaling: how the frequencies are stretched."""
    factor: float
    original: float
    fast: float
    slow: float

    def to_json_dict(self) -> dict:
        return {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}


def stretched_frequencies(base: float, dims: int, s: Optional[StretchConfig]) -> Tuple[List[float], float]:
    """(the dims/2 frequencies, the amplitude of cosine and sine), in 64-bit.  Pair i turns at f_i = base^(-2i/dims).  The
    index at which a pair makes t turns over `original` positions is j(t) = dims ln(original / (2 pi t)) / (2 ln base);
    with lo = max(floor(j(fast)), 0), hi = min(ceil(j(slow)), dims - 1) and r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
    the frequency is r_i f_i / factor + (1 - r_i) f_i, and the amplitude is 0.1 ln(factor) + 1."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if s is None:
        return f, 1.0
    at = lambda turns: dims * math.log(s.original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo, hi = max(math.floor(at(s.fast)), 0), min(math.ceil(at(s.slow)), dims - 1)
    out = []
    for i, fi in enumerate(f):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / s.factor * r + fi * (1.0 - r))
    return out, 0.1 * math.log(s.factor) + 1.0


@dataclass(frozen=True)
class AttentionMixerConfig:
    """The sizes of grouped-query attention; what else a mixer has is None (or 0) where its config.json object lacks it."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int] = None           # mask.size
    rot_base: float = 10000.0
    rot_dims: int = 0                      # 0: no rotation
    stretch: Optional[StretchConfig] = None
    softcap: Optional[float] = None

    def to_json_dict(self) -> dict:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.rot_dims:
            out["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
            if self.stretch is not None:
                out["rot"]["scaling"] = self.stretch.to_json_dict()
        if self.softcap is not None:
            out["softcap"] = self.softcap
        return out


@dataclass(frozen=True)
class DecayMixerConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    def to_json_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: AttentionMixerConfig
    right: DecayMixerConfig
    left_scale: float
    right_scale: float

    def to_json_dict(self) -> dict:
        return {"left": self.left.to_json_dict(), "right": self.right.to_json_dict(), "left_scale": self.left_scale,
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class SofudraLayerConfig:
    type: str                              # "attention" or "parallel"
    mixer: object                          # AttentionMixerConfig or ParallelMixerConfig
    ff: Optional[int]                      # None: no feed-forward


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


def _attention_mixer(f: ConfigFields) -> AttentionMixerConfig:
    heads, kv_heads = _positive(f, "heads"), _positive(f, "kv_heads")
    if heads % kv_heads:
        raise ConfigError(f"{f.origin}: heads={heads} is not a multiple of kv_heads={kv_heads}")
    dim = _positive(f, "dim")
    window = None
    mask = f.mapping("mask")
    if mask is not None:
        window = _positive(mask, "size")
    base, dims, stretch = 10000.0, 0, None
    rot = f.mapping("rot")
    if rot is not None:
        dims = rot.integer("dims", required=True)
        base = rot.number("base", required=True)
        if dims < 0 or dims % 2 or dims > dim:
            raise ConfigError(f"{rot.origin}: dims={dims} must be even and at most dim={dim}")
        if not base > 1.0:
            raise ConfigError(f"{rot.origin}: base={base} must exceed 1")
        sc = rot.mapping("scaling")
        if sc is not None:
            stretch = StretchConfig(factor=sc.number("factor", required=True), original=sc.number("original", required=True),
                                    fast=sc.number("fast", required=True), slow=sc.number("slow", required=True))
            if not (stretch.factor > 0.0 and stretch.original > 0.0 and stretch.fast > 0.0 and stretch.slow > 0.0):
                raise ConfigError(f"{sc.origin}: factor, original, fast and slow must be positive")
    softcap = f.number("softcap")
    if softcap is not None and not softcap > 0.0:
        raise ConfigError(f"{f.origin}: softcap={softcap} must be positive")
    return AttentionMixerConfig(heads=heads, kv_heads=kv_heads, dim=dim, vdim=_positive(f, "vdim"),
                                scale=f.number("scale", required=True), window=window, rot_base=base, rot_dims=dims,
                                stretch=stretch, softcap=softcap)


def _decay_mixer(f: ConfigFields) -> DecayMixerConfig:
    heads = _positive(f, "heads")
    decay = f.number_or_list("decay", required=True)
    if len(decay) == 1:
        decay = decay * heads
    if len(decay) != heads or any(not 0.0 <= d <= 1.0 for d in decay):
        raise ConfigError(f"{f.origin}: 'decay' gives {len(decay)} numbers for {heads} heads, each between 0 and 1")
    return DecayMixerConfig(heads=heads, dim=_positive(f, "dim"), vdim=_positive(f, "vdim"), decay=tuple(decay))


def _parallel_mixer(f: ConfigFields) -> ParallelMixerConfig:
    left, right = f.mapping("left"), f.mapping("right")
    if left is None or right is None:
        raise ConfigError(f"{f.origin} missing 'left' or 'right'")
    return ParallelMixerConfig(left=_attention_mixer(left), right=_decay_mixer(right),
                               left_scale=f.number("left_scale", required=True), right_scale=f.number("right_scale", required=True))


@dataclass(frozen=True)
class SofudraConfig:
    vocab: int
    width: int
    norm_eps: float
    embed_scale: float
    residual_mult: float
    logit_softcap: float                   # 0: logits as they are
    layers: Tuple[SofudraLayerConfig, ...]
    loop: Optional[LoopConfig]

    architecture = "Sofudra"
    model_type = "sofudra"

    @classmethod
    def from_fields(cls, f: ConfigFields, tensor_names: Optional[Iterable[str]] = None) -> "SofudraConfig":
        vocab, width = _positive(f, "vocab"), _positive(f, "width")
        norm = f.mapping("norm")
        if norm is None:
            raise ConfigError(f"{f.origin} missing 'norm'")
        eps = norm.number("eps", required=True)
        if not eps >= 0.0:
            raise ConfigError(f"{f.origin}: norm.eps={eps} must not be negative")
        emb = f.mapping("embedding")
        embed_scale = 1.0 if emb is None else emb.number("scale", 1.0)
        cap = f.number("logit_softcap", 0.0)
        if cap < 0.0:
            raise ConfigError(f"{f.origin}: logit_softcap={cap} must not be negative")
        entries = f.mapping_list("layers", required=True)
        if not entries:
            raise ConfigError(f"{f.origin}: 'layers' is empty")
        layers = []
        for e in entries:
            kind = e.string("type", required=True)
            mf = e.mapping("mixer")
            if mf is None:
                raise ConfigError(f"{e.origin} missing 'mixer'")
            if kind == "attention":
                mixer = _attention_mixer(mf)
            elif kind == "parallel":
                mixer = _parallel_mixer(mf)
            else:
                raise ConfigError(f"{e.origin}: layer type '{kind}' is not known (attention, parallel)")
            mlp, ff = e.mapping("mlp"), None
            if mlp is not None:
                if mlp.string("kind", required=True) != "dense":
                    raise ConfigError(f"{mlp.origin}: feed-forward kind '{mlp.string('kind')}' is not known (dense)")
                ff = _positive(mlp, "ff")
            layers.append(SofudraLayerConfig(type=kind, mixer=mixer, ff=ff))
        loop = None
        lf = f.mapping("loop")
        if lf is not None:
            loop = LoopConfig(start=lf.integer("start", required=True), stop=lf.integer("stop", required=True),
                              times=lf.integer("times", required=True))
            if not 0 <= loop.start <= loop.stop <= len(layers) or loop.times < 1:
                raise ConfigError(f"{lf.origin}: start={loop.start}, stop={loop.stop}, times={loop.times} do not name a run of "
                                  f"the {len(layers)} layers passed at least once")
            if loop.start == loop.stop:
                loop = None
        return cls(vocab=vocab, width=width, norm_eps=eps, embed_scale=embed_scale, residual_mult=f.number("residual_mult", 1.0),
                   logit_softcap=cap, layers=tuple(layers), loop=loop)

    def to_json_dict(self) -> dict:
        """The configuration as config.json keys (what the random-weights mode writes)."""
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "embedding": {"scale": self.embed_scale}, "residual_mult": self.residual_mult,
               "layers": [{"type": l.type, "mixer": l.mixer.to_json_dict(),
                           "mlp": None if l.ff is None else {"kind": "dense", "ff": l.ff}} for l in self.layers]}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return out


def _attention_spec(d: int, m: AttentionMixerConfig, eps: float, *, bias: bool, sink, gate) -> AttentionSpec:
    if m.rot_dims:
        freqs, amp = stretched_frequencies(m.rot_base, m.rot_dims, m.stretch)
        position = PositionSpec(kind="rope", rotary_dim=m.rot_dims, theta=m.rot_base, pairing="split_half",
                                frequencies=tuple(freqs), amplitude=amp)
    else:
        position = PositionSpec(kind="none")
    return AttentionSpec(hidden=d, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, qkv_bias=bias, position=position,
                         window=m.window, scale=m.scale, v_head_dim=m.vdim, qk_norm="head", qk_norm_eps=eps, sink=sink,
                         gate=gate, score_cap=m.softcap)


def _attention_names(prefix: str, to: str, *, bias: bool, sink: bool, gate: bool) -> dict:
    names = {f"{prefix}q_proj.weight": to + "q", f"{prefix}k_proj.weight": to + "k", f"{prefix}v_proj.weight": to + "v",
             f"{prefix}q_norm.weight": to + "q.norm", f"{prefix}k_norm.weight": to + "k.norm", f"{prefix}o_proj.weight": to + "o"}
    if bias:
        names.update({f"{prefix}q_proj.bias": to + "q.b", f"{prefix}k_proj.bias": to + "k.b", f"{prefix}v_proj.bias": to + "v.b"})
    if sink:
        names[f"{prefix}sink"] = to + "sink"
    if gate:
        names[f"{prefix}g_proj.weight"] = to + "g"
    return names


def build_spec(cfg: SofudraConfig) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    layers = []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        names = {"mixer_norm.weight": p + "norm1"}
        if l.type == "attention":
            mixer = _attention_spec(d, l.mixer, eps, bias=False, sink="learned", gate=None)
            names.update(_attention_names("mixer.", p + "mix.", bias=False, sink=True, gate=False))
        else:
            left = _attention_spec(d, l.mixer.left, eps, bias=True, sink=False, gate="head")
            r = l.mixer.right
            right = DecayAttentionSpec(hidden=d, n_heads=r.heads, dim=r.dim, vdim=r.vdim, decay=r.decay, eps=eps)
            mixer = ParallelMixersSpec(hidden=d, branches=(left, right), scales=(l.mixer.left_scale, l.mixer.right_scale),
                                       labels=("left", "right"))
            names.update(_attention_names("mixer.left.", p + "mix.left.", bias=True, sink=False, gate=True))
            for part, short in (("q_proj", "q"), ("k_proj", "k"), ("v_proj", "v"), ("g_proj", "g"), ("o_proj", "o")):
                names[f"mixer.right.{part}.weight"] = f"{p}mix.right.{short}"
            names["mixer.right.norm.weight"] = p + "mix.right.norm"
        parts = {"mixer": mixer, "mixer_norm": NormSpec(size=d, eps=eps)}
        if l.ff is not None:
            parts["feed_forward_norm"] = NormSpec(size=d, eps=eps)
            parts["feed_forward"] = DenseActSpec(hidden=d, intermediate=l.ff, activation="gelu_tanh")
            names.update({"feed_forward_norm.weight": p + "norm2", "feed_forward.up.weight": p + "mlp.up",
                          "feed_forward.down.weight": p + "mlp.down"})
        layers.append(LayerSpec(parts, names, block="parallel" if l.ff is not None else "parallel_mixer",
                                block_args={"residual_mult": cfg.residual_mult}))
    n = len(layers)
    entries = []
    if cfg.loop is None:
        order = [Stage(layer=i) for i in range(n)]
    else:
        entries.append(EntrySpec(part=InputMixSpec(hidden=d), names={"weight": "loop.in"}))
        lo, hi = cfg.loop.start, cfg.loop.stop
        order = [Stage(layer=i) for i in range(lo)]
        for _ in range(cfg.loop.times):            # every pass: caches and states of its own, the input mix in front
            order += [Stage(layer=i, enter=0 if i == lo else None) for i in range(lo, hi)]
        order += [Stage(layer=i) for i in range(hi, n)]
    return ModelSpec(vocab=cfg.vocab, hidden=d, layers=layers, order=order, final_norm=NormSpec(size=d, eps=eps),
                     embed_name="embed", final_norm_name="final.norm", head_name="head", embed_scale=cfg.embed_scale,
                     logit_softcap=cfg.logit_softcap, entries=entries)


ARCHITECTURE = register_architecture(Architecture(
    name=SofudraConfig.architecture, model_type=SofudraConfig.model_type,
    config_class=SofudraConfig, build_spec=build_spec))
