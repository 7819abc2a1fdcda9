"""Routed experts: every token goes through `top` of `experts` small feed-forwards, chosen by the largest router scores.

A step's (token, rank) assignments are laid out expert by expert on the device, the experts' products run as ONE grouped
product each (up with the activation in its epilogue, then down), and the results are added per token in rank order.
Nothing is read back to the host and every grid depends on the step's shapes alone, so the step can be captured.  The
router's logits are float whatever the compute type; its matrix is kept in float32.  A row's result is a function of that
row alone (each output summed over the inner size in index order), so it does not depend on what else the step holds.

Options of the spec: experts with a gate branch and a clamped activation (gate and up as one grouped product, the
activation a kernel between the two products); scores that are a softmax over all router outputs; a learned bias that
takes part in the choice but not in the weights; a constant on the weights; router outputs that stand for experts without
weights, which return their input (their rows of the grouped products stay empty, and the sum per token takes the input
row in their place); a shared expert that every token passes, whose gate/up product also carries, as one more row of its
matrix, the number per token whose sigmoid multiplies its result.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List

import torch

from ..csrc import ops
from .context import BuildContext
from .linear import Linear
from .registry import register_feed_forward
from .spec import RoutedExpertsSpec, TensorRole


@dataclass
class RoutedRows:
    """The experts' results before they are added up per token: rows [T * top, hidden] float32 laid out expert by expert,
    `row_of[t * top + j]` the row of token t's rank j, `weights` the chosen scores, `scale` whether they still multiply.
    A norm that stands behind the experts adds the rows up itself (`RMSNorm.norm_add`)."""
    rows: torch.Tensor
    row_of: torch.Tensor
    weights: torch.Tensor
    top: int
    scale: bool


@register_feed_forward("routed_experts")
class RoutedExperts:
    @staticmethod
    def expected_tensors(spec: RoutedExpertsSpec) -> List[TensorRole]:
        outputs = spec.experts + spec.identity
        roles = [TensorRole("router.weight", (outputs, spec.hidden), True, True)]
        if spec.choice_bias:
            roles.append(TensorRole("router.bias", (outputs,), role="bias"))
        for e in range(spec.experts):
            if spec.activation == "glu_clamped":
                roles.append(TensorRole(f"experts.{e}.gate.weight", (spec.intermediate, spec.hidden), True, True))
            roles += [TensorRole(f"experts.{e}.up.weight", (spec.intermediate, spec.hidden), True, True),
                      TensorRole(f"experts.{e}.down.weight", (spec.hidden, spec.intermediate), True, True)]
        if spec.shared is not None:
            im = spec.shared.intermediate
            roles += [TensorRole("shared.gate.weight", (im, spec.hidden), True, True),
                      TensorRole("shared.up.weight", (im, spec.hidden), True, True),
                      TensorRole("shared.down.weight", (spec.hidden, im), True, True)]
            if spec.shared.gated:
                roles.append(TensorRole("shared.scale.weight", (1, spec.hidden), True, True))
        return roles

    gives_rows = True          # forward(..., summed=False) hands out RoutedRows (the plain form; the extended one sums itself)

    def __init__(self, spec: RoutedExpertsSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        self.glu = spec.activation == "glu_clamped"
        if not self.glu and (spec.activation not in ops.EXPERT_ACTIVATIONS or spec.activation == "none"):
            raise ValueError(f"unknown activation '{spec.activation}' of an expert (relu2, glu_clamped)")
        if spec.router_activation not in ops.ROUTER_MODES:
            raise ValueError(f"unknown router activation '{spec.router_activation}' ({', '.join(ops.ROUTER_MODES)})")
        outputs = spec.experts + spec.identity
        if spec.experts < 1 or spec.identity < 0 or not 1 <= spec.top <= min(outputs, 32):
            raise ValueError(f"top={spec.top} must be between 1 and the number of router outputs ({outputs}), at most 32")
        if (self.glu or spec.shared is not None) and not (spec.limit > 0.0 if self.glu else True):
            raise ValueError("the clamped activation wants a positive limit")
        self.extended = bool(spec.identity or spec.shared is not None or spec.choice_bias or spec.route_scale != 1.0
                             or spec.router_activation == "softmax" or self.glu)
        if self.extended and spec.scale_input:
            raise ValueError("identity experts, a shared expert and the clamped activation weigh the experts' results, not their inputs")
        self.spec, self.ctx = spec, ctx
        f32 = lambda t: t.to(device=ctx.device, dtype=torch.float32).contiguous()
        self.router = f32(tensors["router.weight"])
        self.choice_bias = f32(tensors["router.bias"]) if spec.choice_bias else None
        if self.glu:            # gate above up, per expert: one grouped product for both
            self.up = torch.stack([torch.cat([ctx.matrix(tensors[f"experts.{e}.gate.weight"]),
                                              ctx.matrix(tensors[f"experts.{e}.up.weight"])], dim=0)
                                   for e in range(spec.experts)]).contiguous()
        else:
            self.up = torch.stack([ctx.matrix(tensors[f"experts.{e}.up.weight"]) for e in range(spec.experts)]).contiguous()
        self.down = torch.stack([ctx.matrix(tensors[f"experts.{e}.down.weight"]) for e in range(spec.experts)]).contiguous()
        self.tensor_cores = ctx.gemm != "library"
        self.shared_up = self.shared_down = None
        if spec.shared is not None:
            if not spec.shared.limit > 0.0:
                raise ValueError("the shared expert's clamped activation wants a positive limit")
            rows = [tensors["shared.gate.weight"], tensors["shared.up.weight"]]
            if spec.shared.gated:                  # the number per token rides as one more row; zeros up to a multiple of 8 rows
                w = tensors["shared.scale.weight"].reshape(1, -1)
                rows += [w, torch.zeros((7, w.shape[1]), dtype=w.dtype, device=w.device)]
            self.shared_up = Linear(torch.cat(rows, dim=0), None, ctx, label="proj_gate_up")
            self.shared_down = Linear(tensors["shared.down.weight"], None, ctx, label="proj_down")

    def forward(self, h: torch.Tensor, batch, summed: bool = True):
        """h [T, hidden] in the compute type -> the sum of the chosen experts' results, float32 [T, hidden]; or, with
        `summed` False, the results as `RoutedRows`, for a consumer that adds them up itself."""
        if not isinstance(h, torch.Tensor):
            h = h.tensor()
        s, dev, ct = self.spec, h.device, self.ctx.compute_dtype
        T, A = h.shape[0], h.shape[0] * s.top
        outputs = s.experts + s.identity
        ints = torch.empty((3 * A + outputs + 1,), dtype=torch.int32, device=dev)
        ids, row_of, src_of, offsets = ints[:A].view(T, s.top), ints[A:2 * A], ints[2 * A:3 * A], ints[3 * A:]
        weights = torch.empty((T, s.top), dtype=torch.float32, device=dev)
        ops.route(h, self.router, s.top, ids, weights, sigmoid=s.router_activation, renorm=s.renormalize,
                  bias=self.choice_bias, scale=s.route_scale)
        ops.route_sort(ids.view(-1), outputs, offsets, row_of, src_of)
        if s.identity:                                 # (rows of experts without weights: assigned, never computed)
            offsets = offsets[:s.experts + 1]
        xp = torch.empty((A, s.hidden), dtype=ct, device=dev)
        ops.route_gather(h, weights.view(-1), src_of, xp, s.top, scale=s.scale_input)
        hp = torch.empty((A, s.intermediate), dtype=ct, device=dev)
        if self.glu:
            gu = torch.empty((A, 2 * s.intermediate), dtype=ct, device=dev)
            ops.gemm_grouped(xp, self.up, offsets, gu, "none", self.ctx.status, self.tensor_cores)
            ops.glu_clamped(gu, hp, s.limit)
        else:
            ops.gemm_grouped(xp, self.up, offsets, hp, s.activation, self.ctx.status, self.tensor_cores)
        yp = torch.empty((A, s.hidden), dtype=torch.float32, device=dev)
        ops.gemm_grouped(hp, self.down, offsets, yp, "none", self.ctx.status, self.tensor_cores)
        if not self.extended:
            if not summed:
                return RoutedRows(yp, row_of, weights.view(-1), s.top, not s.scale_input)
            out = torch.empty((T, s.hidden), dtype=torch.float32, device=dev)
            ops.route_combine(yp, weights.view(-1), row_of, out, s.top, scale=not s.scale_input)
            return out
        shared = gate = None
        if s.shared is not None:
            im = s.shared.intermediate
            # [T, gate | up (| the gate's number, zeros)]: float from the fused product of few rows, else in the compute type
            gu = self.shared_up.full_f32(h) if self.shared_up.fuses(T) else self.shared_up(h)
            act = torch.empty((T, im), dtype=ct, device=dev)
            ops.glu_clamped(gu, act, s.shared.limit)
            shared = self.shared_down.full_f32(act)
            gate = gu[:, 2 * im] if s.shared.gated else None
        out = torch.empty((T, s.hidden), dtype=torch.float32, device=dev)
        ops.route_combine_ext(yp, weights.view(-1), row_of, ids.view(-1), s.experts, h, out, s.top, shared=shared, sg=gate)
        return out
