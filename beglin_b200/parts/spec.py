"""Descriptions of the parts a model is put together from.  Pure data: no tensors, no device.

A model is a `ModelSpec`: an embedding, a list of layers, the order in which the layers run, a
final norm and a head.  Every layer names the kind of its block, mixer, feed-forward, norms and
position encoding and gives each its sizes and constants, so two layers of one model may differ in
all of them.  The kinds are looked up in the registries of `beglin_b200.parts.registry`; a spec
never names the architecture it came from.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass(frozen=True)
class TensorRole:
    """One tensor a part wants: its name inside the part, its shape, whether it may be absent,
    whether it is a matrix of a matrix product (kept in the compute dtype) or a small vector or
    table (kept as stored), and what it is for.  `role` decides how random weights are drawn:
    "matrix" and "vector" around zero, "bias" around zero with a deviation of its own, "scale" (a
    norm's weight, which multiplies) around one, "average" (the weights of a sum whose last term is the main
    one) around zero with the last around one.  Empty means "matrix" or "vector" by `matrix`."""
    name: str
    shape: Tuple[int, ...]
    required: bool = True
    matrix: bool = False
    role: str = ""

    def init_role(self) -> str:
        return self.role or ("matrix" if self.matrix else "vector")


@dataclass(frozen=True)
class NormSpec:
    """kind "rmsnorm": x * rsqrt(mean(x^2) + eps) * w.  kind "layernorm": centred first,
    c = x - mean(x), then c * rsqrt(mean(c^2) + eps) * w; there is no shift vector.  `offset` o (rmsnorm): the stored
    weight lies around zero and the rows are multiplied by o + w, the sum formed in float."""
    size: int
    eps: float
    kind: str = "rmsnorm"
    offset: float = 0.0


@dataclass(frozen=True)
class PositionSpec:
    """Rotary position encoding: `rotary_dim` leading features of each head are rotated in pairs,
    (i, i + rotary_dim/2) for pairing "split_half" (qwen_infer.c:782-790) or (2i, 2i+1) for
    "interleaved" (qwen_infer.c:738-750); frequency i is theta^(-2i/rotary_dim) * freq_scale[i]
    (qwen_infer.c:757-794).  kind "none" rotates nothing.  `freq_divisor` d divides every frequency (positions
    stretched d times, "linear scaling"); with it the frequencies are worked out in 64-bit and rounded once.
    `frequencies`, when given, ARE the rotary_dim/2 frequencies (worked out by whoever wrote the spec, in 64-bit; rounded
    once here), and theta, freq_scale and freq_divisor play no part.  `amplitude` multiplies every cosine and sine."""
    kind: str = "rope"
    rotary_dim: int = 0
    theta: float = 10000.0
    pairing: str = "split_half"
    freq_scale: Optional[Tuple[float, ...]] = None
    freq_divisor: Optional[float] = None
    frequencies: Optional[Tuple[float, ...]] = None
    amplitude: float = 1.0


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query attention over a paged cache.  `window` None means all earlier positions; a
    number w means the last w positions, the token itself included.  `own_kv` False makes a mixer
    that projects no keys and values of its own and reads the cache of another stage.

    Options beyond the plain form, each off by default.  `v_head_dim`: values of another size than queries and
    keys (a page then holds the keys of all kv heads followed by their values).  `qk_norm` "projection": the whole
    query row and the whole key row of a token (all heads at once) are RMS-normed with weights of their own,
    before the rotation, with `qk_norm_eps`.  `sink`: the softmax's denominator is enlarged by one, as if every
    query saw one more key of score 0 that carries no value.  `gate` "elementwise": the joined heads are multiplied
    by sigmoid of a further product of the mixer's input, feature by feature, before the output product; `gate` "head": that
    product gives ONE number per query head, whose sigmoid multiplies the head's result.  `qk_norm` "head": every head of
    the queries and of the keys is RMS-normed by itself, with one weight vector of head_dim values for all query heads and one
    for all key heads.  `sink` "learned": the extra key's score is a learned number per query head (tensor `sink`) in place
    of 0.  `score_cap` c: a scaled score s becomes c tanh(s / c) before the softmax.  `block` b (in place of a window): a query
    at position i sees the keys j <= i with floor(j / b) = floor(i / b), blocks counted from position 0 of the sequence."""
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    qkv_bias: bool
    position: PositionSpec
    out_bias: bool = False
    window: Optional[int] = None
    scale: Optional[float] = None          # None: 1/sqrt(head_dim)  (qwen_infer.c:1488)
    own_kv: bool = True
    v_head_dim: Optional[int] = None       # None: head_dim
    qk_norm: Optional[str] = None          # None, "projection" or "head"
    qk_norm_eps: float = 0.0
    sink: object = False                   # False, True (a key of score 0) or "learned" (a score per query head)
    gate: Optional[str] = None             # None, "elementwise" or "head"
    score_cap: Optional[float] = None      # None: scores as they are
    block: Optional[int] = None            # None: no blocks of positions
    kind: str = "gqa_attention"

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else self.v_head_dim


@dataclass(frozen=True)
class SwiGLUSpec:
    """down(act(gate(h)) * up(h)); `activation` "silu" or "gelu_tanh" (the tanh form of GELU)."""
    hidden: int
    intermediate: int
    activation: str = "silu"
    kind: str = "swiglu"


@dataclass(frozen=True)
class RoutedExpertsSpec:
    """A sum over `top` of `experts` small feed-forwards, chosen per token by the largest router scores.  An expert
    is down(act(up(h))) without a gate branch and without biases; `activation` "relu2" is the square of relu.
    `router_activation` "sigmoid": the scores are sigmoid of the router's logits, which are computed in 32-bit.
    `renormalize`: whether the chosen scores are divided by their sum.  `scale_input`: the score multiplies the
    expert's input (True) or its output (False).

    `activation` "glu_clamped": an expert has a gate branch, down(g sigmoid(1.702 g) (u + 1)) with g = min(gate(h), `limit`)
    and u = clamp(up(h), -limit, limit).  `router_activation` "softmax": the scores are the softmax of the logits over all
    router outputs.  `choice_bias`: a learned number per router output (tensor `router.bias`) is added to the scores when
    the experts are chosen, and plays no part in the weights.  `route_scale` multiplies the weights.  `identity` n: the
    router has `experts` + n outputs, and the last n stand for experts without weights that return their input.
    `shared`: an expert that every token passes, added to the sum."""
    hidden: int
    intermediate: int
    experts: int
    top: int
    activation: str = "relu2"
    router_activation: str = "sigmoid"
    renormalize: bool = False
    scale_input: bool = True
    limit: float = 0.0
    choice_bias: bool = False
    route_scale: float = 1.0
    identity: int = 0
    shared: Optional[SharedExpertSpec] = None
    kind: str = "routed_experts"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Attention whose keys and values are made from a cached low-rank latent.  Per head `dim` features that
    are not rotated and `rot_dim` that are (queries), the rotated key part being ONE vector shared by all
    heads; values of `vdim` features; the queries pass a latent of `q_rank` features, keys and values one of
    `kv_rank`.  `position.rotary_dim` leading features of the rot part turn.  Each head's result is scaled by
    sigmoid of a per-head gate read from the mixer's input when `gated`.  `own_kv` False: no down-projection
    of its own; the latent and key part of another stage's cache are read.  `q_rank` None: the queries are one product
    of the mixer's input (tensor `q_proj.weight`), without a latent of their own.  `rot_dim` 0: no rotated part at all.
    `window` w: a query sees itself and the w - 1 positions before it."""
    hidden: int
    n_heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: Optional[int]
    kv_rank: int
    scale: float
    eps: float
    position: PositionSpec
    gated: bool = True
    own_kv: bool = True
    window: Optional[int] = None
    kind: str = "latent_attention"


@dataclass(frozen=True)
class Mamba2Spec:
    """The Mamba-2 recurrence: `n_heads` heads of `vdim` features with a state of `state` x vdim each, B and C
    shared inside each of `groups` groups of heads, a causal convolution of `conv` taps over x, B and C, and
    an RMS norm of the gated result in `norm_groups` equal parts."""
    hidden: int
    n_heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int
    eps: float
    kind: str = "mamba2"


@dataclass(frozen=True)
class DecayAttentionSpec:
    """Linear attention with a constant decay per head: `n_heads` heads with queries and keys of `dim` features and values
    of `vdim`; q, k, v = silu of products of the mixer's input; per head a state S <- decay_h S + k v^T [dim, vdim] that
    is read out as S^T q.  The joined heads are RMS-normed together with a weight (`eps`), multiplied feature by feature by
    sigmoid of a further product of the input, and projected."""
    hidden: int
    n_heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    eps: float
    kind: str = "decay_attention"


@dataclass(frozen=True)
class ParallelMixersSpec:
    """Several mixers side by side that read the same input; the result is sum_i scales[i] * mixer_i(h).  `labels` name the
    branches: branch i's tensors are called `<labels[i]>.<the mixer's own name>`.  Every branch has a cache of its own
    kind (pages, state) or none."""
    hidden: int
    branches: Tuple[object, ...]
    scales: Tuple[float, ...]
    labels: Tuple[str, ...]
    kind: str = "parallel_mixers"


@dataclass(frozen=True)
class InputMixSpec:
    """What stands in front of a stage: the stream is replaced by W [x; e], e the embedded rows of the step and W
    [hidden, 2 hidden] (the stream's half first)."""
    hidden: int
    kind: str = "input_mix"


@dataclass(frozen=True)
class RGLRUSpec:
    """A recurrent block around a real-gated linear recurrent unit.  Two branches of `width` channels: y = gelu_tanh(W_y h +
    b_y), and u = the causal convolution per channel (`conv` taps, a bias, no activation) of W_x h + b_x.  u is cut into
    `blocks` equal parts; in part b, r = sigmoid(A_b u_b + a_b) and i = sigmoid(B_b u_b + b_b) with square matrices.  Per
    channel log a = -`decay_scale` r softplus(lam), S <- a S + sqrt(1 - a^2) (i u) from S = 0 at a request's start, and the
    result is W_o (S * y)."""
    hidden: int
    width: int
    blocks: int
    conv: int
    decay_scale: float = 8.0
    kind: str = "rglru"


@dataclass(frozen=True)
class LaneLinkSpec:
    """How a sublayer is tied to a residual kept in `lanes` copies: it reads sum_a in[a] lane_a, and its result y replaces
    every lane at once, lane_b <- sum_a mix[a, b] lane_a + out[b] y."""
    lanes: int
    kind: str = "lane_link"


@dataclass(frozen=True)
class SharedExpertSpec:
    """An expert of the routed experts' form that every token passes; its result is multiplied by sigmoid of one number per
    token, a product of the feed-forward's input, when `gated`."""
    intermediate: int
    limit: float
    gated: bool = True


@dataclass(frozen=True)
class DenseActSpec:
    """Feed-forward with one hidden layer, down(act(up(h))), no gate branch.  `activation` "xielu": a parabola
    above zero and a scaled exponential below, with two learned numbers (tensor `act`); "gelu_tanh" and "silu" have no
    tensor of their own."""
    hidden: int
    intermediate: int
    activation: str = "xielu"
    kind: str = "dense_act"


@dataclass(frozen=True)
class DepthAverageSpec:
    """Behind a layer the stream is replaced by a learned weighted sum of the embedded rows and every layer's
    result up to this one: `terms` of them for this layer (its own result is the last), out of `total` in the
    model."""
    terms: int
    total: int
    kind: str = "depth_average"


class LayerSpec:
    """One decoder layer: the kind of its block, and the spec of the part in every slot that the block
    kind declares (`parts`: slot name -> part spec; the block class's `SLOTS` says which slots there are
    and of which family each is).  `names` maps each part's own tensor names, qualified by the slot, to
    checkpoint names, e.g. {"mixer.q_proj.weight": "model.layers.3.self_attn.q_proj.weight"}.

    The slots may also be given as keywords (`LayerSpec(mixer=..., feed_forward=..., names=...)`) and
    read as attributes (`layer.mixer`); `with_parts` returns a copy with some slots, the names or the
    block kind replaced.  `block_args` are the constants of the block kind itself (keyword arguments of its class, e.g. the
    factor on the sublayers' sum of a "parallel" block)."""

    def __init__(self, parts: Optional[Dict[str, object]] = None, names: Optional[Dict[str, str]] = None,
                 block: str = "prenorm", block_args: Optional[Dict[str, object]] = None, **slots):
        merged = dict(parts or {})
        merged.update(slots)
        object.__setattr__(self, "parts", merged)
        object.__setattr__(self, "names", dict(names or {}))
        object.__setattr__(self, "block", block)
        object.__setattr__(self, "block_args", dict(block_args or {}))

    def __getattr__(self, slot):
        parts = self.__dict__.get("parts", {})
        if slot in parts:
            return parts[slot]
        raise AttributeError(f"the layer has no slot '{slot}' (slots: {', '.join(parts) or 'none'})")

    def __setattr__(self, key, value):
        raise AttributeError("a LayerSpec is not changed in place; use with_parts()")

    def with_parts(self, names: Optional[Dict[str, str]] = None, block: Optional[str] = None, **slots) -> "LayerSpec":
        parts = dict(self.parts)
        parts.update(slots)
        return LayerSpec(parts, self.names if names is None else names, self.block if block is None else block,
                         self.block_args)

    def __repr__(self):
        return f"LayerSpec(block={self.block!r}, parts={self.parts!r})"


@dataclass(frozen=True)
class Stage:
    """One entry of the run order: which layer runs, and whose cache it uses.  `cache` None means
    a cache of its own; a number names an earlier stage of the order whose cache is read.  `enter` names one of the
    model's `entries`, a part that rewrites the stream right before this stage runs."""
    layer: int
    cache: Optional[int] = None
    enter: Optional[int] = None


@dataclass(eq=False)
class EntrySpec:
    """A part in front of stages (family "entry"): its spec and the checkpoint names of its tensors."""
    part: object
    names: Dict[str, str]


@dataclass
class ModelSpec:
    vocab: int
    hidden: int
    layers: List[LayerSpec]
    order: List[Stage]
    final_norm: NormSpec
    embed_name: str
    final_norm_name: str
    head_name: Optional[str]              # None: the head is the embedding table (tied)
    max_positions: Optional[int] = None
    embed_scale: float = 1.0              # the embedded rows are multiplied by this (1: as they are)
    head_bias_name: Optional[str] = None  # a bias [vocab] added to the logits
    logit_softcap: float = 0.0            # c > 0: logits = c * tanh(logits / c)
    eos_ids: Tuple[int, ...] = ()
    lanes: int = 0                        # n > 0: the residual is kept in n lanes, all equal to the embedded rows at the start;
    #                                       the final norm reads their sum (blocks of a "lanes" kind tie the sublayers to them)
    extra: Dict[str, object] = field(default_factory=dict)
    entries: List[EntrySpec] = field(default_factory=list)   # parts that stages name in `enter`
