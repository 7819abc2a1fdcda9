"""A residual kept in several lanes (hyper-connections), and the blocks that run on it.

The model starts n lanes as copies of the embedded rows (`ModelSpec.lanes`).  A sublayer tied to them by a link with the
constants r [n], M [n, n], w [n] reads z = sum_a r_a lane_a, computes y = sublayer(norm(z)), and y replaces all lanes at
once: lane_b <- sum_a M[a, b] lane_a + w_b y.  The final norm reads the sum of the lanes.  A block of kind "lanes_prenorm"
is the pre-norm layer on such a residual: mixer, then feed-forward, each with a norm and a link of its own.

A sublayer's result stays owed to the lanes until the next read, which is one kernel (`lane_step`): the write of the last
sublayer, the read of the next and its RMS norm in one pass over the lanes.  Lanes, constants, sums and norm are float in
both number formats.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .context import BuildContext
from .registry import register_block, register_link
from .spec import LaneLinkSpec, TensorRole
from .stream import ResidualStream


@register_link("lane_link")
class LaneLink:
    @staticmethod
    def expected_tensors(spec: LaneLinkSpec) -> List[TensorRole]:
        n = spec.lanes
        return [TensorRole("in", (n,), role="scale"), TensorRole("out", (n,), role="scale"),
                TensorRole("mix", (n, n), role="scale")]

    def __init__(self, spec: LaneLinkSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        if not 1 <= spec.lanes <= 8:
            raise ValueError(f"lanes={spec.lanes}: a residual has one to eight lanes")
        self.spec, self.ctx = spec, ctx
        f32 = lambda t: t.to(device=ctx.device, dtype=torch.float32).contiguous()
        self.inw, self.out, self.mix = f32(tensors["in"]), f32(tensors["out"]), f32(tensors["mix"])     # mix [from, to]


@register_block("lanes_prenorm")
class LanesPreNormBlock:
    SLOTS = (("mixer_norm", "norm"), ("mixer_link", "link"), ("mixer", "mixer"),
             ("feed_forward_norm", "norm"), ("feed_forward_link", "link"), ("feed_forward", "feed_forward"))

    def __init__(self, mixer_norm, mixer_link, mixer, feed_forward_norm=None, feed_forward_link=None, feed_forward=None):
        for norm in (mixer_norm, feed_forward_norm):
            if norm is not None and getattr(norm, "kind", None) != "rmsnorm":
                raise ValueError("a block on lanes norms with RMS norms")
        self.mixer_norm, self.mixer_link, self.mixer = mixer_norm, mixer_link, mixer
        self.feed_forward_norm, self.feed_forward_link, self.feed_forward = feed_forward_norm, feed_forward_link, feed_forward

    def forward(self, stream: ResidualStream, batch, cache) -> None:
        if stream.lanes is None:
            raise RuntimeError("a block on lanes runs in a model whose spec keeps its residual in lanes")
        dtype = self.mixer_norm.ctx.compute_dtype
        h = stream.lane_read(self.mixer_link, self.mixer_norm, dtype)
        if getattr(self.mixer, "takes_stream", False):
            y = self.mixer.forward(h, batch, cache, None)
        else:
            y = self.mixer.forward(h, batch, cache)
        stream.lane_owe(y, self.mixer_link)
        if self.feed_forward is not None:
            h = stream.lane_read(self.feed_forward_link, self.feed_forward_norm, dtype)
            if getattr(self.feed_forward, "takes_stream", False):
                y = self.feed_forward.forward(h, batch, None)
            else:
                y = self.feed_forward.forward(h, batch)
            stream.lane_owe(y, self.feed_forward_link)


@register_block("lanes_prenorm_mixer")
class LanesPreNormMixerBlock(LanesPreNormBlock):
    """The same layer without a feed-forward."""
    SLOTS = (("mixer_norm", "norm"), ("mixer_link", "link"), ("mixer", "mixer"))
