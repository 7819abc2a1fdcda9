"""SwiGLU feed-forward: m = W_down (silu(W_gate h) * (W_up h)), no biases (qwen_infer.c:1560-1573,
:727-733).  Gate and up run as one product over the concatenated matrix [2*im, d], as the
reference fuses them (qwen_infer.c:1368-1402).  The spec's `activation` may name the tanh form of GELU in
silu's place; of the products with the activation in their epilogue, the one of many rows (pairs of CTAs) knows both,
the fused one of few rows silu only, so a decoding step with GELU runs the plain product and the activation kernel."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..csrc import ops
from .context import BuildContext
from .linear import Linear
from .registry import register_feed_forward
from .spec import DenseActSpec, SwiGLUSpec, TensorRole
from .stream import ResidualStream


@register_feed_forward("swiglu")
class SwiGLU:
    @staticmethod
    def expected_tensors(spec: SwiGLUSpec) -> List[TensorRole]:
        return [TensorRole("gate_proj.weight", (spec.intermediate, spec.hidden), True, True),
                TensorRole("up_proj.weight", (spec.intermediate, spec.hidden), True, True),
                TensorRole("down_proj.weight", (spec.hidden, spec.intermediate), True, True)]

    takes_stream = True        # forward takes a NormedInput and may add its result to the stream itself

    def __init__(self, spec: SwiGLUSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        if spec.activation not in ops.GLU_ACTIVATIONS:
            raise ValueError(f"unknown activation '{spec.activation}' of a gated feed-forward ({', '.join(ops.GLU_ACTIVATIONS)})")
        self.spec, self.ctx = spec, ctx
        gate, up, im = tensors["gate_proj.weight"], tensors["up_proj.weight"], spec.intermediate
        # Where the intermediate size allows it, the rows go in blocks of 64: gate, up, gate, up, ...  A CTA of
        # the fused product (128 rows) then holds 64 gate features with their 64 up features and applies
        # silu(gate) * up itself; the plain kernel reads the same layout.
        self.block = 64 if im % 64 == 0 else 0
        if self.block:
            w = torch.stack([gate.reshape(im // 64, 64, -1), up.reshape(im // 64, 64, -1)], dim=1).reshape(2 * im, -1)
        else:
            w = torch.cat([gate, up], dim=0)
        self.gate_up = Linear(w, None, ctx, label="proj_gate_up")
        self.down = Linear(tensors["down_proj.weight"], None, ctx, label="proj_down")

    def forward(self, h, batch, stream: Optional[ResidualStream] = None) -> Optional[torch.Tensor]:
        """h: the normed rows, or a NormedInput.  With `stream` the result is added to it (or left owed to
        it) and None is returned; without, the addend is returned."""
        act = self.gate_up.of(h, swiglu=True, activation=self.spec.activation) if self.block else None
        if act is None:
            gu = self.gate_up.of(h)
            act = torch.empty((gu.shape[-2], self.spec.intermediate), dtype=self.ctx.compute_dtype, device=gu.device)
            ops.swiglu(gu, act, self.block, self.spec.activation)
        if stream is None:
            return self.down.partial(act)
        self.down.into(act, stream)
        return None


@register_feed_forward("dense_act")
class DenseAct:
    """m = W_down act(W_up h): one hidden layer without a gate branch.  The activation (xIELU, the tanh form of GELU or
    silu) is a kernel of its own between the two products; it reads the up product's result (or its partial sums) as floats and writes
    the compute type."""

    @staticmethod
    def expected_tensors(spec: DenseActSpec) -> List[TensorRole]:
        roles = [TensorRole("up.weight", (spec.intermediate, spec.hidden), True, True),
                 TensorRole("down.weight", (spec.hidden, spec.intermediate), True, True)]
        if spec.activation == "xielu":
            roles.append(TensorRole("act", (2,)))
        return roles

    def __init__(self, spec: DenseActSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        if spec.activation != "xielu" and spec.activation not in ops.GLU_ACTIVATIONS:
            raise ValueError(f"unknown activation '{spec.activation}' of a dense feed-forward "
                             f"(xielu, {', '.join(ops.GLU_ACTIVATIONS)})")
        self.spec, self.ctx = spec, ctx
        self.up = Linear(tensors["up.weight"], None, ctx, label="proj_up")
        self.down = Linear(tensors["down.weight"], None, ctx, label="proj_down")
        self.act = ctx.vector(tensors["act"]) if spec.activation == "xielu" else None

    takes_stream = True        # forward takes a NormedInput and may add its result to the stream itself

    def forward(self, h, batch, stream: Optional[ResidualStream] = None) -> Optional[torch.Tensor]:
        """h: the normed rows, or a NormedInput.  With `stream` the result is added to it (or left owed to it) and None
        is returned; without, the addend is returned."""
        if not isinstance(h, torch.Tensor):
            h = h.tensor()
        z = self.up.partial(h)
        a = torch.empty((h.shape[0], self.spec.intermediate), dtype=self.ctx.compute_dtype, device=h.device)
        if self.act is not None:
            ops.xielu(z, self.act, a)
        else:
            ops.activation(z, a, self.spec.activation)
        if stream is None:
            return self.down.partial(a)
        self.down.into(a, stream)
        return None
