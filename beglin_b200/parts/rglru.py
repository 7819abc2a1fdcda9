"""A recurrent block around a real-gated linear recurrent unit (RG-LRU).

One product of the mixer's input gives both branches side by side, [y | x]; their biases are added where its rows are read.  x passes a short causal
convolution per channel (no activation) and becomes u; u is cut into equal parts, and in each part two square matrices
give the gates, r = sigmoid(A_b u_b + a_b) and i = sigmoid(B_b u_b + b_b).  Per channel
    log a = -C r softplus(lam),   S <- e^(log a) S + sqrt(1 - e^(2 log a)) (i u),
from S = 0 at a request's start, and the result is W_o (S * gelu_tanh(y)).

The state S and the last taps - 1 inputs of the convolution are per-request state of fixed size (one slot of the cache
manager's slab, float32, zero when the request starts): a step continues each request from its slot, however the request's
tokens are cut into steps and whatever else the step holds.  Everything that enters the recurrence is float in both number
formats: the input product comes out as float, the convolution, the gates' products, sigmoids, softplus, decay, step and
state are float.  The gates' products run on the CUDA cores in float32 steps (every output summed in index order); in
bfloat16 steps on the tensor cores, with u cut into two bfloat16 numbers that together hold sixteen bits of it, against the
matrices in bfloat16, accumulated in float.  Portions of at least `CHUNK_FROM` rows of a request walk
the recurrence in chunks that are joined by a scan over the chunks' (product of decays, sum); shorter ones and single
tokens walk it row by row, so two ways of cutting a prompt differ by the rounding of those sums.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..csrc import ops
from .cache_need import FixedStateNeed, FixedStateView
from .context import BuildContext
from .linear import Linear
from .registry import register_mixer
from .spec import RGLRUSpec, TensorRole
from .stream import NormedInput, ResidualStream


@register_mixer("rglru")
class RGLRU:
    CHUNK_FROM = 64            # a request that brings at least this many rows walks them in chunks
    CHUNK_ROWS = 32

    @staticmethod
    def expected_tensors(spec: RGLRUSpec) -> List[TensorRole]:
        W, d, B = spec.width, spec.hidden, spec.blocks
        bs = W // max(B, 1)
        return [TensorRole("y_proj.weight", (W, d), True, True), TensorRole("y_proj.bias", (W,), role="bias"),
                TensorRole("x_proj.weight", (W, d), True, True), TensorRole("x_proj.bias", (W,), role="bias"),
                TensorRole("conv.weight", (W, spec.conv)), TensorRole("conv.bias", (W,), role="bias"),
                TensorRole("gate_r.weight", (B, bs, bs), True, True), TensorRole("gate_r.bias", (B, bs), role="bias"),
                TensorRole("gate_i.weight", (B, bs, bs), True, True), TensorRole("gate_i.bias", (B, bs), role="bias"),
                TensorRole("lam", (W,)),
                TensorRole("o_proj.weight", (d, W), True, True)]

    @staticmethod
    def cache_need(spec: RGLRUSpec) -> FixedStateNeed:
        return FixedStateNeed((spec.width * spec.conv,), "float32")        # S (width) and taps - 1 rows of inputs

    def __init__(self, spec: RGLRUSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        if spec.blocks < 1 or spec.width % spec.blocks:
            raise ValueError(f"{spec.width} channels do not fall into {spec.blocks} equal parts")
        if spec.conv < 1:
            raise ValueError("the convolution has at least one tap")
        self.spec, self.ctx = spec, ctx
        W = spec.width
        f32 = lambda t: t.to(device=ctx.device, dtype=torch.float32).contiguous()
        # (the branches' biases are added where the product's rows are read: by the convolution and by the walk)
        self.in_proj = Linear(torch.cat([tensors["y_proj.weight"], tensors["x_proj.weight"]], dim=0), None, ctx, label="proj_in")
        self.bias_y, self.bias_x = f32(tensors["y_proj.bias"]), f32(tensors["x_proj.bias"])
        self.o_proj = Linear(tensors["o_proj.weight"], None, ctx, label="proj_o")
        self.conv_w, self.conv_b = f32(tensors["conv.weight"]), f32(tensors["conv.bias"])
        # per part the two gates' matrices one above the other: [blocks, 2 bs, bs], float
        self.gate_w = f32(torch.cat([tensors["gate_r.weight"], tensors["gate_i.weight"]], dim=1))
        # bfloat16 steps: the gates' products on the tensor cores, from u cut into two bfloat16 numbers (sixteen bits of it)
        # against the matrices in bfloat16 repeated along the inner size; accumulation and result are float
        self.gate_w2 = None
        if ctx.compute_dtype == torch.bfloat16 and (W // spec.blocks) % 8 == 0:
            w = ctx.matrix(self.gate_w)
            self.gate_w2 = torch.cat([w, w], dim=2).transpose(1, 2).contiguous()      # [blocks, 2 bs (inner), 2 bs (out)]
        self.bias_r, self.bias_i = f32(tensors["gate_r.bias"]).view(-1), f32(tensors["gate_i.bias"]).view(-1)
        self.decay = torch.empty((W,), dtype=torch.float32, device=ctx.device)
        with torch.cuda.device(ctx.device):
            ops.rglru_softplus(tensors["lam"].to(ctx.device).contiguous(), spec.decay_scale, self.decay)

    takes_stream = True        # forward takes a NormedInput and may add its result to the stream itself

    def forward(self, h, batch, cache: FixedStateView, stream: Optional[ResidualStream] = None) -> Optional[torch.Tensor]:
        """h: the normed rows, or a NormedInput.  With `stream` the result is added to it (or left owed to it) and None
        is returned; without, the addend is returned."""
        if isinstance(h, NormedInput):
            h = h.tensor()
        s, ctx = self.spec, self.ctx
        T, W, B = batch.n_rows, s.width, s.blocks
        proj = self.in_proj.full_f32(h)                                 # [T, y | x] without their biases
        reqs, n_req = batch.query_blocks(1 << 30)                       # one (request, first row, rows) per request
        u = torch.empty((T, W), dtype=torch.float32, device=h.device)
        ops.conv_silu(proj, W, W, self.conv_w, self.conv_b, cache.state, W, cache.slots, batch.row_req, reqs, n_req, u,
                      activation="none", src_bias=self.bias_x)
        if self.gate_w2 is not None:
            x2 = torch.empty((B, T, 2 * (W // B)), dtype=torch.bfloat16, device=h.device)
            ops.rglru_split(u, B, x2)
            with ops.phase("proj_heads"):
                gates = torch.bmm(x2, self.gate_w2, out_dtype=torch.float32)
        else:
            gates = torch.empty((B, T, 2 * (W // B)), dtype=torch.float32, device=h.device)
            ops.gemm_f32_nt_batched(u.view(T, B, W // B).transpose(0, 1), self.gate_w, gates)
        out = torch.empty((T, W), dtype=ctx.compute_dtype, device=h.device)
        if max(batch.lens) < self.CHUNK_FROM:
            ops.rglru_scan(gates, u, proj, 0, self.bias_r, self.bias_i, self.decay, cache.state, cache.slots, reqs, n_req, out,
                           y_bias=self.bias_y)
        else:
            short, n_short, chunks, n_chunks, longs, n_long = batch.long_blocks(self.CHUNK_ROWS, self.CHUNK_FROM)
            if n_short:
                ops.rglru_scan(gates, u, proj, 0, self.bias_r, self.bias_i, self.decay, cache.state, cache.slots, short, n_short, out,
                               y_bias=self.bias_y)
            ops.rglru_scan(gates, u, proj, 0, self.bias_r, self.bias_i, self.decay, cache.state, cache.slots, None, 0, out,
                           chunked=(chunks, n_chunks, longs, n_long, self.CHUNK_ROWS), y_bias=self.bias_y)
        if stream is None:
            return self.o_proj.partial(out)
        self.o_proj.into(out, stream)
        return None
