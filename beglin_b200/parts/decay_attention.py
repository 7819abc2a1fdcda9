"""Linear attention with a constant decay per head.

One product of the mixer's input gives, side by side, the rows for q, k, v and the gate g.  With q, k, v = silu of their
rows, per head h and for each token in turn
    S <- d_h S + k v^T;    o = S^T q
(S of `dim` x `vdim` values, d_h a constant of the head).  The joined heads o are RMS-normed over the whole row with a
weight, multiplied feature by feature by sigmoid(g), and go through the output product.

The state S is per-request state of fixed size (one slot of the cache manager's slab, float32, zero when the request
starts): a step continues each request from its slot, however the request's tokens are cut into steps and whatever else
the step holds.  State, decay, the products that enter the state and the readout are float in both number formats.

A request that brings many rows runs in chunks of tokens: with S the state at a chunk's start and t, j counting the
chunk's r tokens from 0, o_t = d^(t+1) S^T q_t + sum_{j <= t} d^(t-j) (q_t . k_j) v_j and the state behind the chunk is
d^r S + sum_j d^(r-1-j) k_j v_j^T, so the chunks' own sums and outputs are computed side by side and only a pass over
the chunks' states is serial.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..csrc import ops
from .cache_need import FixedStateNeed, FixedStateView
from .context import BuildContext
from .linear import Linear
from .registry import register_mixer
from .spec import DecayAttentionSpec, TensorRole
from .stream import NormedInput, ResidualStream


@register_mixer("decay_attention")
class DecayAttention:
    @staticmethod
    def expected_tensors(spec: DecayAttentionSpec) -> List[TensorRole]:
        qd, vd = spec.n_heads * spec.dim, spec.n_heads * spec.vdim
        return [TensorRole("q_proj.weight", (qd, spec.hidden), True, True),
                TensorRole("k_proj.weight", (qd, spec.hidden), True, True),
                TensorRole("v_proj.weight", (vd, spec.hidden), True, True),
                TensorRole("g_proj.weight", (vd, spec.hidden), True, True),
                TensorRole("norm.weight", (vd,), role="scale"),
                TensorRole("o_proj.weight", (spec.hidden, vd), True, True)]

    @staticmethod
    def cache_need(spec: DecayAttentionSpec) -> FixedStateNeed:
        return FixedStateNeed((spec.n_heads * spec.dim * spec.vdim,), "float32")

    def __init__(self, spec: DecayAttentionSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        if len(spec.decay) != spec.n_heads:
            raise ValueError(f"{len(spec.decay)} decays for {spec.n_heads} heads")
        if any(not 0.0 <= float(d) <= 1.0 for d in spec.decay):
            raise ValueError("a decay lies between 0 and 1")
        self.spec, self.ctx = spec, ctx
        self.qd, self.vd = spec.n_heads * spec.dim, spec.n_heads * spec.vdim
        w = torch.cat([tensors[n + ".weight"] for n in ("q_proj", "k_proj", "v_proj", "g_proj")], dim=0)
        self.in_proj = Linear(w, None, ctx, label="proj_qkv")
        self.o_proj = Linear(tensors["o_proj.weight"], None, ctx, label="proj_o")
        self.norm_w = ctx.vector(tensors["norm.weight"])
        self.decay = torch.tensor([float(d) for d in spec.decay], dtype=torch.float32, device=ctx.device)
        self.g_col = 2 * self.qd + self.vd
        self.chunk = ops.decay_attention_chunk(spec.dim, spec.vdim) if ctx.device.type == "cuda" else 0

    LONG_FROM = 16             # rows of a request in a step from which its tokens run in chunks

    takes_stream = True        # forward takes a NormedInput and may add its result to the stream itself

    def forward(self, h, batch, cache: FixedStateView, stream: Optional[ResidualStream] = None) -> Optional[torch.Tensor]:
        """h: the normed rows, or a NormedInput.  With `stream` the result is added to it (or left owed to it) and None
        is returned; without, the addend is returned."""
        if isinstance(h, NormedInput):
            h = h.tensor()
        s = self.spec
        T = batch.n_rows
        proj = self.in_proj(h, out_dtype=torch.float32)                 # [T, q | k | v | g]
        y = torch.empty((T, self.vd), dtype=torch.float32, device=h.device)
        if self.chunk and not batch.decode_only and hasattr(batch, "long_blocks"):
            # requests of LONG_FROM rows and more in chunks, the others token by token
            reqs, n_req, chunks, n_chunks, longs, n_long = batch.long_blocks(self.chunk, self.LONG_FROM)
        else:
            reqs, n_req = batch.query_blocks(1 << 30)                   # one (request, first row, rows) per request
            chunks, n_chunks, longs, n_long = None, 0, None, 0
        ops.decay_attention(proj, 0, self.qd, 2 * self.qd, self.decay, cache.state, cache.slots, reqs, n_req, y,
                            s.n_heads, s.dim, s.vdim, chunks, n_chunks, longs, n_long)
        out = torch.empty((T, self.vd), dtype=self.ctx.compute_dtype, device=h.device)
        ops.gated_group_rmsnorm(y, proj, self.g_col, self.norm_w, s.eps, 1, out, gate_after=True)
        if stream is None:
            return self.o_proj.partial(out)
        self.o_proj.into(out, stream)
        return None
