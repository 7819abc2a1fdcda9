"""The arrangement of a layer's parts.  "prenorm" is the reference's decoder layer:
h = norm(x); x += mixer(h); h = norm(x); x += feed_forward(h)  (qwen_infer.c:1447, :1552, :1556,
:1577).  The residual x is float.  A block does not add its last result to x itself: it returns it,
and the next norm (of the next block, or the final one) adds it, fused with its statistics; or, in
steps of few tokens, the part's last product adds it and the next part's first product norms (see
stream.py).  The other kinds are the same layer without a feed-forward, and either with a combiner
behind it: a part that rewrites the stream from the results of this and earlier layers."""
from __future__ import annotations

import torch

from ..csrc import ops
from .registry import register_block
from .stream import NormedInput, ResidualStream, Terms


@register_block("prenorm")
class PreNormBlock:
    # the slots of a layer of this kind, in the order they are built: (slot name, family of the part).  A
    # block is constructed with one keyword argument per slot.
    SLOTS = (("mixer_norm", "norm"), ("mixer", "mixer"), ("feed_forward_norm", "norm"), ("feed_forward", "feed_forward"))

    def __init__(self, mixer_norm, mixer, feed_forward_norm=None, feed_forward=None, combiner=None):
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.feed_forward_norm, self.feed_forward = feed_forward_norm, feed_forward
        self.combiner = combiner

    def forward(self, stream: ResidualStream, batch, cache) -> None:
        """Runs the layer on the residual stream.  A part that declares `takes_stream` gets the norm of the
        stream uncomputed (its first product may apply it) and the stream itself (its last product may add
        to it); any other part gets the normed rows and returns its addend, which the stream then owes.
        A combiner sees the stream before the sublayers (`begin`) and rewrites it behind them (`forward`)."""
        if self.combiner is not None:
            stream.settle()
            self.combiner.begin(stream)
        h = NormedInput(stream, self.mixer_norm)
        if getattr(self.mixer, "takes_stream", False):
            a = self.mixer.forward(h, batch, cache, stream)
        else:
            a = self.mixer.forward(h.tensor(), batch, cache)
        if a is not None:
            stream.owe(a)
        if self.feed_forward is not None:
            h = NormedInput(stream, self.feed_forward_norm)
            if getattr(self.feed_forward, "takes_stream", False):
                m = self.feed_forward.forward(h, batch, stream)
            else:
                m = self.feed_forward.forward(h.tensor(), batch)
            if m is not None:
                stream.owe(m)
        if self.combiner is not None:
            self.combiner.forward(stream, batch)


@register_block("prenorm_mixer")
class PreNormMixerBlock(PreNormBlock):
    """A layer without a feed-forward: x += mixer(norm(x)) and nothing else."""
    SLOTS = (("mixer_norm", "norm"), ("mixer", "mixer"))


@register_block("prenorm_combined")
class PreNormCombinedBlock(PreNormBlock):
    """The pre-norm layer with a combiner behind it (e.g. the depth-weighted average of the layer results)."""
    SLOTS = PreNormBlock.SLOTS + (("combiner", "combiner"),)


@register_block("prenorm_mixer_combined")
class PreNormMixerCombinedBlock(PreNormBlock):
    SLOTS = PreNormMixerBlock.SLOTS + (("combiner", "combiner"),)


@register_block("postnorm")
class PostNormBlock:
    """The norm stands on a sublayer's RESULT, not on its input: x += norm(mixer(x)), then x += norm(feed_forward(x)).
    The sublayers read the stream as it is: the float rows themselves in the float32 path, their rounding to the
    compute type otherwise (left behind by the kernel that last added to the stream, so no kernel runs for it
    except before a model's first layer).  The statistics of the norm and the sum are float."""
    SLOTS = (("mixer", "mixer"), ("mixer_norm", "norm"), ("feed_forward", "feed_forward"), ("feed_forward_norm", "norm"))

    def __init__(self, mixer, mixer_norm, feed_forward=None, feed_forward_norm=None):
        self.mixer, self.mixer_norm = mixer, mixer_norm
        self.feed_forward, self.feed_forward_norm = feed_forward, feed_forward_norm

    @staticmethod
    def rows(stream: ResidualStream, dtype: torch.dtype) -> torch.Tensor:
        """The stream's rows in the compute type."""
        stream.settle()
        if stream.pending is not None:                 # something an earlier block of another kind still owes
            ops.add_residual(stream.x, stream.pending)
            stream.updated(None)
        if dtype == torch.float32:
            return stream.x
        if stream.lowp is None:
            stream.lowp = torch.empty(stream.x.shape, dtype=dtype, device=stream.x.device)
            ops.cast_rows(stream.x, stream.lowp)
        return stream.lowp

    def forward(self, stream: ResidualStream, batch, cache) -> None:
        dtype = self.mixer_norm.ctx.compute_dtype
        a = self.mixer.forward(self.rows(stream, dtype), batch, cache)
        stream.updated(None, self.mixer_norm.norm_add(stream.x, a, want_lowp=True))
        if self.feed_forward is not None:
            if getattr(self.feed_forward, "gives_rows", False) and hasattr(self.feed_forward_norm, "norm_add"):
                m = self.feed_forward.forward(self.rows(stream, dtype), batch, summed=False)    # the norm adds the experts' rows up
            else:
                m = self.feed_forward.forward(self.rows(stream, dtype), batch)
            stream.updated(None, self.feed_forward_norm.norm_add(stream.x, m, want_lowp=True))


@register_block("postnorm_mixer")
class PostNormMixerBlock(PostNormBlock):
    """The same layer without a feed-forward."""
    SLOTS = (("mixer", "mixer"), ("mixer_norm", "norm"))


@register_block("parallel")
class ParallelBlock:
    """Both sublayers read the SAME stream, each through a norm of its own, and their sum is added times a constant:
    x <- x + m (mixer(norm1(x)) + feed_forward(norm2(x))); a layer may lack the feed-forward.  The sum is float.  The
    block leaves its sublayers' results as terms that the stream still owes, and the next block of this kind adds them
    in the same kernel that computes its two norms (one pass over the rows for the sum, the statistics and both normed
    copies); any other reader of the stream has them added first."""
    SLOTS = (("mixer_norm", "norm"), ("mixer", "mixer"), ("feed_forward_norm", "norm"), ("feed_forward", "feed_forward"))

    def __init__(self, mixer_norm, mixer, feed_forward_norm=None, feed_forward=None, residual_mult: float = 1.0):
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.feed_forward_norm, self.feed_forward = feed_forward_norm, feed_forward
        self.mult = float(residual_mult)

    def normed(self, stream: ResidualStream):
        """(norm1(x), norm2(x) or None) of the stream with everything it is owed added."""
        n1, n2 = self.mixer_norm, self.feed_forward_norm if self.feed_forward is not None else None
        one_kernel = getattr(n1, "kind", None) == "rmsnorm" and (n2 is None or (
            getattr(n2, "kind", None) == "rmsnorm" and n2.spec.eps == n1.spec.eps and n2.weight.dtype == n1.weight.dtype))
        if not one_kernel:
            stream.settle()
            h1 = NormedInput(stream, n1).tensor()
            return h1, (n2.add_norm(stream.x, None) if n2 is not None else None)
        terms = stream.terms.items if stream.terms is not None else []
        if stream.pending is not None:
            terms = [(stream.pending, 1.0)] + list(terms)
        x, dtype = stream.x, n1.ctx.compute_dtype
        h1 = torch.empty(x.shape, dtype=dtype, device=x.device)
        h2 = torch.empty(x.shape, dtype=dtype, device=x.device) if n2 is not None else None
        ops.add_terms_norm(x, terms, weight1=n1.weight, weight2=n2.weight if n2 is not None else None, eps=n1.spec.eps,
                           out1=h1, out2=h2)
        stream.pending, stream.terms, stream.ssq, stream.lowp = None, None, None, None
        return h1, h2

    def forward(self, stream: ResidualStream, batch, cache) -> None:
        h1, h2 = self.normed(stream)
        owed = Terms()
        if getattr(self.mixer, "takes_stream", False):
            owed.add(self.mixer.forward(h1, batch, cache, None), self.mult)
        else:
            owed.add(self.mixer.forward(h1, batch, cache), self.mult)
        if self.feed_forward is not None:
            if getattr(self.feed_forward, "takes_stream", False):
                owed.add(self.feed_forward.forward(h2, batch, None), self.mult)
            else:
                owed.add(self.feed_forward.forward(h2, batch), self.mult)
        stream.terms = owed


@register_block("parallel_mixer")
class ParallelMixerBlock(ParallelBlock):
    """The same layer without a feed-forward: x <- x + m mixer(norm1(x))."""
    SLOTS = (("mixer_norm", "norm"), ("mixer", "mixer"))
