"""Attention through a low-rank latent, with an output gate per head.

Of every position only ONE row is cached for all heads: the RMS-normed latent c (kv_rank features) and the
rotated key part k_r (rot_dim features) that the heads share.  A head's keys W_uk c and values W_uv c are
never made.  Since q . (W_uk c) = (W_uk^T q) . c, the un-rotated part of a query is carried into the latent
space (one small product per head), the attention kernel scores it against the cached c directly and
returns, per head, the softmax-weighted sum of the c, and W_uv is applied to that sum (again one small
product per head).  So a step never touches more of the cache than the cached rows themselves, whatever the
number of heads.

A step: ONE product of the mixer's input for the query latent, the key/value latent with the key part and
the gates (the matrices are concatenated at load time, with rows of zeros up to a multiple of 16 outputs);
ONE kernel for the norm of the query latent and the norm, rotation and append of the key/value latent; the
query product; queries into the latent space; attention (the queries' rotated part turned inside the kernel)
and the merge of its splits; values out of the latent space; gates; the output product, which in steps of
few rows adds into the residual stream itself.  A mixer with `own_kv` False has no key/value projection and
reads the cache of the stage it is told to.  Options of the spec: queries that are one product of the input (no query
latent), no rotated part, no gates, a sliding window.

Long prompt portions in bfloat16 go the other way round where the sizes allow it (dim + rot_dim = vdim = 64 or
128): the keys and values of all heads are made once per step from the request's cached rows, by ONE product
with [W_uk; W_uv], laid out as pages of a pool of the step's own, and the grouped-query kernel on the tensor
cores (tcgen05) runs over them with one kv head per query head.  Per key and head that is dim + rot_dim + vdim
features instead of 2 kv_rank + rot_dim, at matrix speed; the cache keeps holding the latent rows only.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np
import torch

from ..csrc import ops
from .cache_need import PagedKVView, PagedLatentNeed
from .context import BuildContext
from .linear import Linear
from .registry import register_mixer
from .rope import shared_position
from .spec import LatentAttentionSpec, TensorRole
from .stream import NormedInput, ResidualStream


@register_mixer("latent_attention")
class LatentAttention:
    @staticmethod
    def expected_tensors(spec: LatentAttentionSpec) -> List[TensorRole]:
        H, qd = spec.n_heads, spec.dim + spec.rot_dim
        if spec.q_rank is None:                     # queries straight from the mixer's input
            roles = [TensorRole("q_proj.weight", (H * qd, spec.hidden), True, True)]
        else:
            roles = [TensorRole("q_down.weight", (spec.q_rank, spec.hidden), True, True),
                     TensorRole("q_down.norm", (spec.q_rank,), role="scale"),
                     TensorRole("q_up.weight", (H * qd, spec.q_rank), True, True)]
        roles += [TensorRole("k_up.weight", (H * spec.dim, spec.kv_rank), True, True),
                  TensorRole("v_up.weight", (H * spec.vdim, spec.kv_rank), True, True),
                  TensorRole("o_proj.weight", (spec.hidden, H * spec.vdim), True, True)]
        if spec.own_kv:
            roles += [TensorRole("kv_down.weight", (spec.kv_rank + spec.rot_dim, spec.hidden), True, True),
                      TensorRole("kv_down.norm", (spec.kv_rank,), role="scale")]
        if spec.gated:
            roles.append(TensorRole("gate.weight", (H, spec.hidden), True, True))
        return roles

    @staticmethod
    def cache_need(spec: LatentAttentionSpec) -> Optional[PagedLatentNeed]:
        if not spec.own_kv:
            return None
        return PagedLatentNeed(spec.kv_rank + spec.rot_dim, spec.window)

    def __init__(self, spec: LatentAttentionSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        H = spec.n_heads
        self.position = shared_position(spec.position, ctx)
        self.rot_dims = int(self.position.rotary_dim)
        if self.rot_dims > spec.rot_dim or (self.rot_dims and not self.position.interleaved):
            raise ValueError(f"the rotated part of {spec.rot_dim} features turns in neighbouring pairs over at most "
                             f"its own width, not {self.rot_dims} features paired '{spec.position.pairing}'")
        # the products of the mixer's input, as ONE: [query latent | key/value latent, key part | gates]
        self.direct_q = spec.q_rank is None
        if self.direct_q and not spec.own_kv:
            raise ValueError("latent attention without a query latent has a key/value latent of its own")
        self.q_rank = 0 if self.direct_q else int(spec.q_rank)
        self.window = int(spec.window) if spec.window else 0
        names = ([] if self.direct_q else ["q_down.weight"]) + (["kv_down.weight"] if spec.own_kv else []) \
            + (["gate.weight"] if spec.gated else [])
        w_down = torch.cat([tensors[n] for n in names], dim=0)
        if w_down.shape[0] % 16:                    # rows of zeros up to a multiple of 16 outputs: a width that is no multiple
            pad = 16 - w_down.shape[0] % 16         # of 8 takes the library's product of many rows off its fast kernels
            w_down = torch.cat([w_down, torch.zeros((pad, w_down.shape[1]), dtype=w_down.dtype, device=w_down.device)], dim=0)
        self.down = Linear(w_down, None, ctx, label="proj_qkv")
        self.kv_col = self.q_rank
        self.gate_col = self.q_rank + (spec.kv_rank + spec.rot_dim if spec.own_kv else 0)
        self.q_norm = None if self.direct_q else ctx.vector(tensors["q_down.norm"])
        self.kv_norm = ctx.vector(tensors["kv_down.norm"]) if spec.own_kv else None
        self.q_up = Linear(tensors["q_proj.weight" if self.direct_q else "q_up.weight"], None, ctx, label="proj_q")
        # per head: W_uk^T as [kv_rank, dim] (the product into the latent space is x W^T with W = W_uk^T) and
        # W_uv as [vdim, kv_rank]
        self.k_up_t = ctx.matrix(tensors["k_up.weight"].reshape(H, spec.dim, spec.kv_rank).transpose(1, 2))
        self.v_up = ctx.matrix(tensors["v_up.weight"].reshape(H, spec.vdim, spec.kv_rank))
        self.o_proj = Linear(tensors["o_proj.weight"], None, ctx, label="proj_o")
        self.scale = float(np.float32(spec.scale))
        rows, self.tile = ops.latent_attention_plan(spec.kv_rank, spec.rot_dim)
        self.hc = min(H, rows)                      # heads per CTA
        self.bq = max(1, rows // self.hc)           # rows of one request per CTA
        self.f32 = ctx.compute_dtype == torch.float32
        # bfloat16 steps score on the tensor cores where the cached row's sizes allow it (mma.sync); float32 steps and
        # other sizes on the CUDA cores
        self.mma = None
        if not self.f32 and ctx.cache_dtype == torch.bfloat16 and ctx.attention != "generic":
            plan = ops.latent_attention_mma_plan(spec.kv_rank, spec.rot_dim)
            if plan is not None:
                rows, stages = plan
                hc = min(H, rows)
                self.mma = (hc, max(1, rows // hc), stages)
        # the tensor-core way for long portions: head sizes that the grouped-query kernel takes, bfloat16 throughout
        self.expand = None
        hd = spec.dim + spec.rot_dim
        if not self.f32 and ctx.cache_dtype == torch.bfloat16 and spec.vdim == hd and hd in (64, 128) \
                and spec.dim % 8 == 0 and spec.rot_dim % 8 == 0 \
                and ctx.attention in ("auto", "tcgen05"):
            kernel, bq, tile = ops.attention_plan(1, hd, torch.bfloat16, False, ctx.attention, 64)
            if kernel == "tc_rows":
                self.expand = (bq, tile)
                self.kv_up = ctx.matrix(torch.cat([tensors["k_up.weight"], tensors["v_up.weight"]], dim=0))

    EXPAND_ROWS = 128          # portions of one request of at least this many rows make per-head keys and values

    def _per_head(self, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """out[h] = x[h] @ w[h]^T for x [H, T, K] (a view of any strides) and w [H, N, K]: [H, T, N]."""
        H, T, _ = x.shape
        if self.f32:
            out = torch.empty((H, T, w.shape[1]), dtype=torch.float32, device=x.device)
            ops.gemm_f32_nt_batched(x, w, out)
            return out
        with ops.phase("proj_heads"):
            if out_dtype == x.dtype:
                return torch.bmm(x, w.transpose(1, 2))
            return torch.bmm(x, w.transpose(1, 2), out_dtype=out_dtype)

    def _per_head_keys(self, q: torch.Tensor, down: torch.Tensor, cos_sin, batch, cache: PagedKVView) -> torch.Tensor:
        """The gated heads [T, H vdim] of a portion of ONE request, through keys and values made per head."""
        s, ctx = self.spec, self.ctx
        T, H, hd = batch.n_rows, s.n_heads, s.dim + s.rot_dim
        # every position the portion's rows may see, from the page in which the first row's window begins
        first = 0
        if self.window and batch.starts is not None:                    # (a replayed graph does not know where it stands)
            first = max(0, batch.starts[0] - self.window + 1) // 64 * 64
        S = batch.max_position + 1 - first
        lat = torch.empty((S, s.kv_rank), dtype=torch.bfloat16, device=q.device)
        kr = torch.empty((S, max(s.rot_dim, 8)), dtype=torch.bfloat16, device=q.device)[:, :s.rot_dim]
        ops.latent_gather(cache.pool, cache.block_table, 0, s.kv_rank, lat, kr, first=first)
        with ops.phase("kv_expand"):
            kv = torch.mm(lat, self.kv_up.t())                          # [S, H dim | H vdim]
        pages = torch.empty((-(-S // 64), 2, H, 64, hd), dtype=torch.bfloat16, device=q.device)
        pages[-1].zero_()                                               # what lies behind position S - 1 in the last page
        ops.latent_expand(kv, kr, H, s.dim, pages)
        if self.rot_dims:
            ops.rotate_q(q, H, hd, s.dim, self.rot_dims, cos_sin)
        table = torch.arange(-(first // 64), pages.shape[0], dtype=torch.int32, device=q.device).clamp_(min=-1).view(1, -1)
        bq, tile = self.expand
        qblk, n_qblk = batch.query_blocks(bq)
        att = torch.empty((T, H * hd), dtype=torch.bfloat16, device=q.device)
        ops.attention(q, q.stride(0), pages, table, batch.positions, qblk, n_qblk, batch.max_position, T, H, H, hd, self.window,
                      ctx.kv_split, tile, bq, self.scale, att, ctx.status, "tc_rows")
        if not s.gated:
            return att
        out = torch.empty((T, H * hd), dtype=torch.bfloat16, device=q.device)
        ops.gate_heads(att.view(T, H, hd).transpose(0, 1), down, self.gate_col, out)
        return out

    takes_stream = True        # forward takes a NormedInput and may add its result to the stream itself

    def forward(self, h, batch, cache: PagedKVView, stream: Optional[ResidualStream] = None) -> Optional[torch.Tensor]:
        """h: the normed rows, or a NormedInput.  With `stream` the result is added to it (in steps of few tokens by the
        output product itself) or left owed to it, and None is returned; without, the addend is returned."""
        if isinstance(h, NormedInput):
            h = h.tensor()
        s, ctx = self.spec, self.ctx
        T, H = batch.n_rows, s.n_heads
        down = self.down.full_f32(h)                                    # [T, q_rank (+ kv_rank + rot) (+ H)]
        cos_sin = self.position.table(batch) if self.rot_dims else None
        if self.direct_q:
            ops.latent_append(down, self.kv_col, s.kv_rank, s.rot_dim, self.rot_dims, self.kv_norm, s.eps, cos_sin,
                              batch.positions, batch.row_req, cache.block_table, cache.pool, ctx.status)
            q = self.q_up(h)                                            # [T, H (dim + rot)] straight from the input
        else:
            cq = torch.empty((T, s.q_rank), dtype=ctx.compute_dtype, device=h.device)
            if s.own_kv:                                                # both norms of the product's rows in one launch
                ops.latent_append(down, self.kv_col, s.kv_rank, s.rot_dim, self.rot_dims, self.kv_norm, s.eps, cos_sin,
                                  batch.positions, batch.row_req, cache.block_table, cache.pool, ctx.status,
                                  q_norm=(0, self.q_norm, cq))
            else:
                ops.rmsnorm_slice(down, 0, s.q_rank, self.q_norm, s.eps, cq)
            q = self.q_up(cq)                                           # [T, H (dim + rot)]
        if self.expand is not None and batch.n_req == 1 and T >= self.EXPAND_ROWS:
            return self._result(self._per_head_keys(q, down, cos_sin, batch, cache), stream)
        q_plain = q.view(T, H, s.dim + s.rot_dim)[:, :, :s.dim].transpose(0, 1)          # [H, T, dim]
        q_lat = self._per_head(q_plain, self.k_up_t, torch.float32)    # [H, T, kv_rank] float
        hc, bq, stages = (self.hc, self.bq, 0) if self.mma is None else self.mma
        if getattr(batch, "decode_only", False):
            bq = 1                                                      # one row per request: a CTA's rows are its heads
        qblk, n_qblk = batch.query_blocks(bq)
        if qblk is None:                                                # a decoding graph's batch keeps its list implicit
            batch.implicit_blocks = False
            qblk, n_qblk = batch.query_blocks(bq)
        split = ctx.kv_split
        o_lat = torch.empty((H, T, s.kv_rank), dtype=ctx.compute_dtype, device=h.device)
        ops.latent_attention(q_lat, q, s.dim, s.rot_dim, self.rot_dims, cos_sin, cache.pool, cache.block_table,
                             batch.positions, qblk, n_qblk, batch.max_position, bq, hc, self.tile, split,
                             self.scale, o_lat, ctx.status, mma_stages=stages, window=self.window)
        v = self._per_head(o_lat, self.v_up, ctx.compute_dtype)        # [H, T, vdim]
        out = torch.empty((T, H * s.vdim), dtype=ctx.compute_dtype, device=h.device)
        ops.gate_heads(v, down if s.gated else None, self.gate_col, out)      # (without gates: the heads row by row)
        return self._result(out, stream)

    def _result(self, heads: torch.Tensor, stream: Optional[ResidualStream]) -> Optional[torch.Tensor]:
        if stream is None:
            return self.o_proj.partial(heads)
        self.o_proj.into(heads, stream)
        return None
