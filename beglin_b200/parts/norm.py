"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * weight, statistics in float, eps inside the root, the
weight multiplying directly (qwen_infer.c:711-714), or, with the spec's `offset`, offset + weight.  The residual add that precedes a norm is fused
into it: `add_norm` first does x += delta.  LayerNorm is the same with the mean taken off first and
the variance in place of the mean square; it has a scale vector and no shift."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..csrc import ops
from .context import BuildContext
from .registry import register_norm
from .spec import NormSpec, TensorRole


@register_norm("rmsnorm")
class RMSNorm:
    @staticmethod
    def expected_tensors(spec: NormSpec) -> List[TensorRole]:
        return [TensorRole("weight", (spec.size,), role="vector" if spec.offset else "scale")]

    def __init__(self, spec: NormSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        if spec.offset:                    # a weight stored around zero: offset + w, formed in float and kept so
            self.weight = (tensors["weight"].to(device=ctx.device, dtype=torch.float32) + float(spec.offset)).contiguous()
        else:
            self.weight = ctx.vector(tensors["weight"])
        self._weight_f32 = None

    def weight_f32(self) -> torch.Tensor:
        """The multiplying weight as float32 (for kernels that norm in float from float weights)."""
        if self._weight_f32 is None:
            self._weight_f32 = self.weight if self.weight.dtype == torch.float32 else self.weight.float().contiguous()
        return self._weight_f32

    def add_norm(self, x: torch.Tensor, delta: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None,
                 update: bool = True) -> torch.Tensor:
        """x is the float residual [T, size].  x += delta (when given and `update`), then the normed
        rows in the compute type.  With `rows`, only those rows are normed and x is left alone."""
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.spec.size), dtype=self.ctx.compute_dtype, device=x.device)
        ops.add_rmsnorm(x, delta, self.weight, self.spec.eps, out, rows=rows, update=update and rows is None)
        return out

    def norm_add(self, x: torch.Tensor, y: torch.Tensor, want_lowp: bool = False) -> Optional[torch.Tensor]:
        """The norm on a sublayer's RESULT: x += norm(y) * weight, for y [T, size] or its float partial sums
        [parts, T, size]; statistics and sum in float.  With `want_lowp` the new rows of x are also returned in
        the compute type (for the next sublayer, which reads the stream as it is)."""
        lowp = None
        if want_lowp and self.ctx.compute_dtype != torch.float32:
            lowp = torch.empty(x.shape, dtype=self.ctx.compute_dtype, device=x.device)
        if hasattr(y, "row_of"):               # the results of routed experts, not yet added up per token
            ops.rmsnorm_add_routed(x, y.rows, y.row_of, y.weights, y.top, y.scale, self.weight, self.spec.eps, lowp)
        else:
            ops.rmsnorm_add(x, y, self.weight, self.spec.eps, lowp)
        return lowp

    def fusion(self):
        """What a product needs to apply this norm to its operand itself: (weight, eps); None when the
        weight is not in the compute type (a checkpoint that stores it in 32-bit keeps it so)."""
        if self.weight.dtype != self.ctx.compute_dtype:
            return None
        return self.weight, float(self.spec.eps)


@register_norm("layernorm")
class LayerNorm:
    @staticmethod
    def expected_tensors(spec: NormSpec) -> List[TensorRole]:
        return [TensorRole("weight", (spec.size,), role="scale")]

    def __init__(self, spec: NormSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        self.weight = ctx.vector(tensors["weight"])

    def add_norm(self, x: torch.Tensor, delta: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None,
                 update: bool = True) -> torch.Tensor:
        """As RMSNorm.add_norm: x += delta (when given and `update`), then the normed rows in the compute type."""
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.spec.size), dtype=self.ctx.compute_dtype, device=x.device)
        ops.add_layernorm(x, delta, self.weight, self.spec.eps, out, rows=rows, update=update and rows is None)
        return out
