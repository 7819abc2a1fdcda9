"""The Tuzupel decoder: its configuration, read from the keys of its own config.json, and its description as a list of
parts.

config.json names the architecture in the string `architecture`, gives `vocab`, `width`, `norm.eps`, `streams` (the number
of lanes n the residual is kept in; absent: one plain residual), `logit_softcap` (c tanh(logits / c)) and lists the layers
one by one: each entry gives `type` (which mixer), `mixer` (its sizes and constants) and `mlp` (routed experts, or null for
a layer without a feed-forward).  A layer is pre-norm, mixer then feed-forward; every norm is an RMS norm whose stored
weight lies around zero (the rows are multiplied by 1 + w).  With lanes, a sublayer reads sum_a in[a] lane_a and its result
y replaces the lanes all at once, lane_b <- sum_a mix[a, b] lane_a + out[b] y (tensors `l<i>.hc1.*` for the mixer,
`l<i>.hc2.*` for the feed-forward); the final norm reads the sum of the lanes.  Tensors of layer i are called `l<i>.*`.

Mixers.  "attention": grouped-query attention without biases, every head of queries and keys RMS-normed by itself (one
plain weight vector for all heads), the leading `rot.dims` features of every head turned in neighbouring pairs with
frequencies rescaled band by band (`rot.scaling` {factor, low, high, original}), a query seeing the keys of its own block
of `mask.size` positions only, and a softmax whose denominator also holds exp of a learned number per head.
"latent_attention": keys and values made from one RMS-normed row of `kv_rank` features per position, queries straight from
the input, no positions, a sliding window of `mask.size`.  "rglru": two branches of `width` channels around a gated linear
recurrence per channel, with a causal convolution of `conv` taps and gates in `blocks` parts.

Feed-forward (`mlp.kind` "moe"): `router.experts` experts with a gate branch and a clamped activation (`expert.ff`,
`expert.limit`), of which a token uses `router.top`; the scores are a softmax over all router outputs, a learned correction
joins them for the choice only, the weights are the scores times `router.scale`; the last `router.identity` router outputs
are experts that return their input; `shared`: an expert of the same form for every token, times sigmoid of one number per
token.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Iterable, List, Optional, Tuple

from ..config.reader import ConfigError, ConfigFields
from ..config.registry import Architecture, register_architecture
from ..parts.spec import (AttentionSpec, LaneLinkSpec, LatentAttentionSpec, LayerSpec, ModelSpec, NormSpec, PositionSpec,
                          RGLRUSpec, RoutedExpertsSpec, SharedExpertSpec, Stage)

DECAY_SCALE = 8.0              # log a = -DECAY_SCALE r softplus(lam): fixed by the design


def _positive(f: ConfigFields, key: str) -> int:
    v = f.integer(key, required=True)
    if v <= 0:
        raise ConfigError(f"{f.origin}: {key}={v} must be positive")
    return v


def _window(f: ConfigFields) -> Optional[int]:
    mask = f.mapping("mask")
    return None if mask is None else _positive(mask, "size")


@dataclass(frozen=True)
class BandScaling:
    """rot.scaling: how the frequencies are rescaled by wavelength."""
    factor: float
    low: float
    high: float
    original: float

    def to_json_dict(self) -> dict:
        return {"factor": self.factor, "low": self.low, "high": self.high, "original": self.original}


def banded_frequencies(base: float, dims: int, s: Optional[BandScaling]) -> List[float]:
    """The dims/2 frequencies in 64-bit.  Pair i turns at f = base^(-2i/dims), wavelength l = 2 pi / f.  With a scaling: f
    stays where l < original/high, becomes f / factor where l > original/low, and between the two is the blend
    (1 - t) f / factor + t f with t = (original / l - low) / (high - low)."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if s is not None:
            wavelength = 2.0 * math.pi / f
            if wavelength > s.original / s.low:
                f = f / s.factor
            elif not wavelength < s.original / s.high:
                t = (s.original / wavelength - s.low) / (s.high - s.low)
                f = (1.0 - t) * f / s.factor + t * f
        out.append(f)
    return out


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    block: Optional[int] = None            # mask.size: the block of positions a query stays in
    rot_base: float = 10000.0
    rot_dims: int = 0                      # 0: no rotation
    scaling: Optional[BandScaling] = None

    def to_json_dict(self) -> dict:
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.block is not None:
            out["mask"] = {"size": self.block}
        if self.rot_dims:
            out["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
            if self.scaling is not None:
                out["rot"]["scaling"] = self.scaling.to_json_dict()
        return out


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: Optional[int] = None           # mask.size

    def to_json_dict(self) -> dict:
        out = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "kv_rank": self.kv_rank, "scale": self.scale}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        return out


@dataclass(frozen=True)
class RecurrentMixerConfig:
    width: int
    blocks: int
    conv: int

    def to_json_dict(self) -> dict:
        return {"width": self.width, "blocks": self.blocks, "conv": self.conv}


@dataclass(frozen=True)
class ExpertsConfig:
    ff: int
    limit: float
    experts: int
    top: int
    scale: float
    identity: int = 0
    correction: bool = True                # whether the folder has the choice bias
    shared_ff: Optional[int] = None        # None: no shared expert
    shared_limit: float = 0.0

    def to_json_dict(self) -> dict:
        out = {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit},
               "router": {"experts": self.experts, "identity": self.identity, "scale": self.scale, "top": self.top}}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return out


@dataclass(frozen=True)
class TuzupelLayerConfig:
    type: str                              # "attention", "latent_attention" or "rglru"
    mixer: object
    mlp: Optional[ExpertsConfig]


def _attention_mixer(f: ConfigFields) -> AttentionMixerConfig:
    heads, kv_heads = _positive(f, "heads"), _positive(f, "kv_heads")
    if heads % kv_heads:
        raise ConfigError(f"{f.origin}: heads={heads} is not a multiple of kv_heads={kv_heads}")
    dim = _positive(f, "dim")
    base, dims, scaling = 10000.0, 0, None
    rot = f.mapping("rot")
    if rot is not None:
        dims = rot.integer("dims", required=True)
        base = rot.number("base", required=True)
        if dims < 0 or dims % 2 or dims > dim:
            raise ConfigError(f"{rot.origin}: dims={dims} must be even and at most dim={dim}")
        if not base > 0.0:
            raise ConfigError(f"{rot.origin}: base={base} must be positive")
        sc = rot.mapping("scaling")
        if sc is not None:
            scaling = BandScaling(factor=sc.number("factor", required=True), low=sc.number("low", required=True),
                                  high=sc.number("high", required=True), original=sc.number("original", required=True))
            if not (scaling.factor > 0.0 and scaling.low > 0.0 and scaling.high > 0.0 and scaling.original > 0.0):
                raise ConfigError(f"{sc.origin}: factor, low, high and original must be positive")
    return AttentionMixerConfig(heads=heads, kv_heads=kv_heads, dim=dim, vdim=_positive(f, "vdim"),
                                scale=f.number("scale", required=True), block=_window(f), rot_base=base, rot_dims=dims,
                                scaling=scaling)


def _latent_mixer(f: ConfigFields) -> LatentMixerConfig:
    return LatentMixerConfig(heads=_positive(f, "heads"), dim=_positive(f, "dim"), vdim=_positive(f, "vdim"),
                             kv_rank=_positive(f, "kv_rank"), scale=f.number("scale", required=True), window=_window(f))


def _recurrent_mixer(f: ConfigFields) -> RecurrentMixerConfig:
    width, blocks = _positive(f, "width"), _positive(f, "blocks")
    if width % blocks:
        raise ConfigError(f"{f.origin}: width={width} does not fall into blocks={blocks} equal parts")
    return RecurrentMixerConfig(width=width, blocks=blocks, conv=_positive(f, "conv"))


def _experts(f: ConfigFields, correction: bool) -> ExpertsConfig:
    kind = f.string("kind", required=True)
    if kind != "moe":
        raise ConfigError(f"{f.origin}: feed-forward kind '{kind}' is not known (moe)")
    expert, router = f.mapping("expert"), f.mapping("router")
    if expert is None or router is None:
        raise ConfigError(f"{f.origin} missing 'expert' or 'router'")
    experts, top = _positive(router, "experts"), _positive(router, "top")
    identity = router.integer("identity", 0)
    if identity < 0 or top > experts + identity:
        raise ConfigError(f"{router.origin}: top={top} of {experts} experts and {identity} identity experts")
    limit = expert.number("limit", required=True)
    if not limit > 0.0:
        raise ConfigError(f"{expert.origin}: limit={limit} must be positive")
    shared = f.mapping("shared")
    shared_ff, shared_limit = None, 0.0
    if shared is not None:
        shared_ff, shared_limit = _positive(shared, "ff"), shared.number("limit", required=True)
        if not shared_limit > 0.0:
            raise ConfigError(f"{shared.origin}: limit={shared_limit} must be positive")
    return ExpertsConfig(ff=_positive(expert, "ff"), limit=limit, experts=experts, top=top, scale=router.number("scale", 1.0),
                         identity=identity, correction=correction, shared_ff=shared_ff, shared_limit=shared_limit)


_MIXERS = {"attention": _attention_mixer, "latent_attention": _latent_mixer, "rglru": _recurrent_mixer}


@dataclass(frozen=True)
class TuzupelConfig:
    vocab: int
    width: int
    norm_eps: float
    lanes: int                             # 0: one plain residual
    logit_softcap: float                   # 0: logits as they are
    layers: Tuple[TuzupelLayerConfig, ...]

    architecture = "Tuzupel"
    model_type = "tuzupel"

    @classmethod
    def from_fields(cls, f: ConfigFields, tensor_names: Optional[Iterable[str]] = None) -> "TuzupelConfig":
        vocab, width = _positive(f, "vocab"), _positive(f, "width")
        norm = f.mapping("norm")
        if norm is None:
            raise ConfigError(f"{f.origin} missing 'norm'")
        eps = norm.number("eps", required=True)
        if not eps >= 0.0:
            raise ConfigError(f"{f.origin}: norm.eps={eps} must not be negative")
        lanes = f.integer("streams", 0)
        if not 0 <= lanes <= 8:
            raise ConfigError(f"{f.origin}: streams={lanes} must be between 1 and 8")
        cap = f.number("logit_softcap", 0.0)
        if cap < 0.0:
            raise ConfigError(f"{f.origin}: logit_softcap={cap} must not be negative")
        entries = f.mapping_list("layers", required=True)
        if not entries:
            raise ConfigError(f"{f.origin}: 'layers' is empty")
        names = None if tensor_names is None else set(tensor_names)
        layers = []
        for i, e in enumerate(entries):
            kind = e.string("type", required=True)
            mf = e.mapping("mixer")
            if mf is None:
                raise ConfigError(f"{e.origin} missing 'mixer'")
            if kind not in _MIXERS:
                raise ConfigError(f"{e.origin}: layer type '{kind}' is not known ({', '.join(_MIXERS)})")
            mlp = e.mapping("mlp")
            correction = names is None or f"l{i}.mlp.correction" in names
            layers.append(TuzupelLayerConfig(type=kind, mixer=_MIXERS[kind](mf),
                                             mlp=None if mlp is None else _experts(mlp, correction)))
        return cls(vocab=vocab, width=width, norm_eps=eps, lanes=lanes, logit_softcap=cap, layers=tuple(layers))

    def to_json_dict(self) -> dict:
        """The configuration as config.json keys (what the random-weights mode writes)."""
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": [{"type": l.type, "mixer": l.mixer.to_json_dict(),
                           "mlp": None if l.mlp is None else l.mlp.to_json_dict()} for l in self.layers]}
        if self.lanes:
            out["streams"] = self.lanes
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        return out


def _mixer(d: int, kind: str, m, eps: float, p: str):
    """(mixer spec, its tensors' checkpoint names) of a layer whose tensors begin with `p`."""
    to = p + "mix."
    if kind == "attention":
        if m.rot_dims:
            position = PositionSpec(kind="rope", rotary_dim=m.rot_dims, theta=m.rot_base, pairing="interleaved",
                                    frequencies=tuple(banded_frequencies(m.rot_base, m.rot_dims, m.scaling)))
        else:
            position = PositionSpec(kind="none")
        spec = AttentionSpec(hidden=d, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, qkv_bias=False, position=position,
                             scale=m.scale, v_head_dim=m.vdim, qk_norm="head", qk_norm_eps=eps, sink="learned", block=m.block)
        names = {"mixer.q_proj.weight": to + "q", "mixer.k_proj.weight": to + "k", "mixer.v_proj.weight": to + "v",
                 "mixer.q_norm.weight": to + "q.norm", "mixer.k_norm.weight": to + "k.norm", "mixer.o_proj.weight": to + "o",
                 "mixer.sink": to + "sink"}
        return spec, names
    if kind == "latent_attention":
        spec = LatentAttentionSpec(hidden=d, n_heads=m.heads, dim=m.dim, rot_dim=0, vdim=m.vdim, q_rank=None, kv_rank=m.kv_rank,
                                   scale=m.scale, eps=eps, position=PositionSpec(kind="none"), gated=False, window=m.window)
        names = {"mixer.q_proj.weight": to + "q", "mixer.kv_down.weight": to + "dkv", "mixer.kv_down.norm": to + "dkv.norm",
                 "mixer.k_up.weight": to + "uk", "mixer.v_up.weight": to + "uv", "mixer.o_proj.weight": to + "o"}
        return spec, names
    spec = RGLRUSpec(hidden=d, width=m.width, blocks=m.blocks, conv=m.conv, decay_scale=DECAY_SCALE)
    names = {"mixer.y_proj.weight": to + "y", "mixer.y_proj.bias": to + "y.b", "mixer.x_proj.weight": to + "x",
             "mixer.x_proj.bias": to + "x.b", "mixer.conv.weight": to + "conv", "mixer.conv.bias": to + "conv.b",
             "mixer.gate_r.weight": to + "ra", "mixer.gate_r.bias": to + "ra.b", "mixer.gate_i.weight": to + "ri",
             "mixer.gate_i.bias": to + "ri.b", "mixer.lam": to + "lam", "mixer.o_proj.weight": to + "o"}
    return spec, names


def _feed_forward(d: int, f: ExpertsConfig, p: str):
    to = p + "mlp."
    shared = None if f.shared_ff is None else SharedExpertSpec(intermediate=f.shared_ff, limit=f.shared_limit, gated=True)
    spec = RoutedExpertsSpec(hidden=d, intermediate=f.ff, experts=f.experts, top=f.top, activation="glu_clamped",
                             router_activation="softmax", renormalize=False, scale_input=False, limit=f.limit,
                             choice_bias=f.correction, route_scale=f.scale, identity=f.identity, shared=shared)
    names = {"feed_forward.router.weight": to + "router"}
    if f.correction:
        names["feed_forward.router.bias"] = to + "correction"
    for e in range(f.experts):
        for part in ("gate", "up", "down"):
            names[f"feed_forward.experts.{e}.{part}.weight"] = f"{to}e{e}.{part}"
    if shared is not None:
        names.update({"feed_forward.shared.gate.weight": to + "shared.gate", "feed_forward.shared.up.weight": to + "shared.up",
                      "feed_forward.shared.down.weight": to + "shared.down", "feed_forward.shared.scale.weight": to + "shared.sg"})
    return spec, names


def build_spec(cfg: TuzupelConfig) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    norm = NormSpec(size=d, eps=eps, offset=1.0)
    layers = []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        mixer, names = _mixer(d, l.type, l.mixer, eps, p)
        parts = {"mixer_norm": norm, "mixer": mixer}
        names["mixer_norm.weight"] = p + "norm1"
        if cfg.lanes:
            parts["mixer_link"] = LaneLinkSpec(lanes=cfg.lanes)
            names.update({"mixer_link.in": p + "hc1.in", "mixer_link.out": p + "hc1.out", "mixer_link.mix": p + "hc1.mix"})
        if l.mlp is not None:
            ff, ff_names = _feed_forward(d, l.mlp, p)
            parts.update({"feed_forward_norm": norm, "feed_forward": ff})
            names.update(ff_names)
            names["feed_forward_norm.weight"] = p + "norm2"
            if cfg.lanes:
                parts["feed_forward_link"] = LaneLinkSpec(lanes=cfg.lanes)
                names.update({"feed_forward_link.in": p + "hc2.in", "feed_forward_link.out": p + "hc2.out",
                              "feed_forward_link.mix": p + "hc2.mix"})
        block = ("lanes_prenorm" if cfg.lanes else "prenorm") + ("" if l.mlp is not None else "_mixer")
        layers.append(LayerSpec(parts, names, block=block))
    return ModelSpec(vocab=cfg.vocab, hidden=d, layers=layers, order=[Stage(layer=i) for i in range(len(layers))],
                     final_norm=norm, embed_name="embed", final_norm_name="final.norm", head_name="head",
                     logit_softcap=cfg.logit_softcap, lanes=cfg.lanes)


ARCHITECTURE = register_architecture(Architecture(
    name=TuzupelConfig.architecture, model_type=TuzupelConfig.model_type,
    config_class=TuzupelConfig, build_spec=build_spec))
