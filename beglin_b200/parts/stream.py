"""The float residual of a step and what is still owed to it.

A block's parts hand their results to the stream in one of two ways.  The plain way: the part
returns an addend (a tensor, or the partial sums of a split-K product) and the stream keeps it as
`pending` until the next norm adds it, fused with its statistics.  The fused way, for steps of few
tokens: the part's last product adds its result to `x` itself and leaves the sums of squares of the
new rows in `ssq`, and the next part's first product takes `x` and `ssq` and norms its operand on
the fly; then neither the addend nor the normed rows ever reach global memory, and two kernels of
the layer (the norms) and their launches are gone.
"""
from __future__ import annotations

from typing import Optional

import torch


class Terms:
    """Results that are to be added to the stream, each times a constant: [(tensor or partial sums, constant), ...]."""

    def __init__(self, items=None):
        self.items = list(items or [])

    def add(self, tensor, scale: float = 1.0) -> None:
        if isinstance(tensor, Terms):
            self.items += [(t, c * scale) for t, c in tensor.items]
        elif tensor is not None:
            self.items.append((tensor, float(scale)))

    def scaled(self, scale: float) -> "Terms":
        return Terms([(t, c * scale) for t, c in self.items])


class ResidualStream:
    def __init__(self, x: torch.Tensor):
        self.x = x                                     # float32 [T, d]
        self.pending: Optional[torch.Tensor] = None    # not yet added to x: [T, d] or partial sums [parts, T, d]
        self.ssq: Optional[torch.Tensor] = None        # float32 [parts, >= T]: partial sums of squares of x's rows
        self.history: Optional[torch.Tensor] = None    # float32 [slots, T, d]: the embedding output and the layer
        #                                                results so far, kept by a combiner that mixes over depth
        self.lowp: Optional[torch.Tensor] = None       # x's rows in the compute type, as the kernel that last changed
        #                                                x left them (for sublayers that read the stream un-normed)
        self.terms: Optional[Terms] = None             # not yet added to x either: results with constants of their own
        #                                                (a block that adds scaled sums; whoever reads x calls settle())
        self.origin: Optional[torch.Tensor] = None     # float32 [T, d]: the embedded rows, kept for parts that mix them in
        self.lanes: Optional[torch.Tensor] = None      # float32 [n, T, d]: the residual as n lanes (then x is not the residual)
        self.lane_owed = None                          # (result, link) of the last sublayer, not yet written to the lanes

    # ------------------------------------------------------------------ a residual kept in lanes
    def open_lanes(self, n: int) -> None:
        """Every lane starts as a copy of x."""
        from ..csrc import ops
        self.lanes = torch.empty((n,) + tuple(self.x.shape), dtype=torch.float32, device=self.x.device)
        ops.lane_fill(self.x, self.lanes)
        self.lane_owed = None

    def _owed_args(self) -> dict:
        if self.lane_owed is None:
            return {}
        y, link = self.lane_owed
        return {"owed": y, "mix": link.mix, "out_weights": link.out}

    def lane_read(self, link, norm, dtype: torch.dtype) -> torch.Tensor:
        """What a sublayer tied by `link` reads, RMS-normed by `norm`, in `dtype`; the last sublayer's result is written
        to the lanes in the same pass."""
        from ..csrc import ops
        h = torch.empty(self.x.shape, dtype=dtype, device=self.x.device)
        ops.lane_step(self.lanes, in_weights=link.inw, norm_weight=norm.weight_f32(), eps=norm.spec.eps, h=h, **self._owed_args())
        self.lane_owed = None
        return h

    def lane_owe(self, y: torch.Tensor, link) -> None:
        self.lane_owed = (y, link)

    def lane_sum(self, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The sum of the lanes, float32, with what is owed counted in: of all rows (the lanes are then brought up to
        date) or of `rows` only (they are left as they are)."""
        from ..csrc import ops
        n = self.x.shape[0] if rows is None else rows.numel()
        z = torch.empty((n, self.x.shape[1]), dtype=torch.float32, device=self.x.device)
        ops.lane_step(self.lanes, z=z, rows=rows, **self._owed_args())
        if rows is None:
            self.lane_owed = None
        return z

    def settle(self) -> None:
        """Adds the scaled terms that are still owed to x (the blocks that leave such terms fold the sum into their own
        next kernel; every other reader of x calls this first)."""
        if self.terms is not None:
            from ..csrc import ops
            ops.add_terms_norm(self.x, self.terms.items)
            self.terms, self.ssq, self.lowp = None, None, None

    def owe(self, addend: torch.Tensor) -> None:
        self.pending, self.ssq, self.lowp = addend, None, None

    def updated(self, ssq: Optional[torch.Tensor], lowp: Optional[torch.Tensor] = None) -> None:
        """x was changed in place by a kernel, which left these sums of squares and this copy in the compute type."""
        self.pending, self.ssq, self.lowp = None, ssq, lowp


class NormedInput:
    """norm(stream) that has not been computed: a part whose first product can norm its operand takes
    it as it is (`Linear.of`); any other part asks for `tensor()`."""

    def __init__(self, stream: ResidualStream, norm):
        self.stream, self.norm = stream, norm
        self._tensor: Optional[torch.Tensor] = None

    @property
    def rows(self) -> int:
        return self.stream.x.shape[0]

    def tensor(self) -> torch.Tensor:
        if self._tensor is None:
            s = self.stream
            s.settle()
            had = s.pending is not None
            self._tensor = self.norm.add_norm(s.x, s.pending)
            s.pending = None
            if had:
                s.ssq = None                            # x has changed
        return self._tensor

    def fusable(self):
        """(weight, eps) of the norm when a product may apply it to the stream itself, else None."""
        s = self.stream
        if self._tensor is not None or s.pending is not None or s.terms is not None or s.ssq is None:
            return None
        return getattr(self.norm, "fusion", lambda: None)()
