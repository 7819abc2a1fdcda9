"""Parts that rewrite the stream in front of a stage (family "entry").

"input_mix": x <- W [x; e], with e the embedded rows of the step and W [hidden, 2 hidden] whose first half of columns
meets the stream.  It stands in front of every pass of a run of layers that is repeated with the same weights.  The
product is split in its halves, W [x; e] = W_x x + W_e e: the second term is the same for every pass of a step and is
computed once; the sum of the two is float and becomes the new stream.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..csrc import ops
from .context import BuildContext
from .linear import Linear
from .registry import register_entry
from .spec import InputMixSpec, TensorRole
from .stream import ResidualStream


@register_entry("input_mix")
class InputMix:
    needs_origin = True        # the model keeps the embedded rows in stream.origin

    @staticmethod
    def expected_tensors(spec: InputMixSpec) -> List[TensorRole]:
        return [TensorRole("weight", (spec.hidden, 2 * spec.hidden), True, True)]

    def __init__(self, spec: InputMixSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        w, d = tensors["weight"], spec.hidden
        self.of_stream = Linear(w[:, :d].contiguous(), None, ctx, label="proj_in")
        self.of_origin = Linear(w[:, d:].contiguous(), None, ctx, label="proj_in")

    def _rows(self, x: torch.Tensor) -> torch.Tensor:
        if self.ctx.compute_dtype == torch.float32:
            return x
        low = torch.empty(x.shape, dtype=self.ctx.compute_dtype, device=x.device)
        ops.cast_rows(x, low)
        return low

    def forward(self, stream: ResidualStream, batch) -> None:
        stream.settle()
        if stream.pending is not None:
            ops.add_residual(stream.x, stream.pending)
            stream.updated(None)
        key = ("input_mix", id(self))
        fixed = batch.scratch.get(key)
        if fixed is None:                     # W_e e: once per step
            fixed = batch.scratch[key] = self.of_origin.partial(self._rows(stream.origin))
        moving = self.of_stream.partial(stream.lowp if stream.lowp is not None else self._rows(stream.x))
        ops.add_terms_norm(stream.x, [(moving, 1.0), (fixed, 1.0)], assign=True)
        stream.updated(None)
