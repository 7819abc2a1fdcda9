"""Grouped-query attention over the paged cache (the reference's attention, qwen_infer.c:1451-1548
for one token and :2075-2136 for a ragged batch).

Per step: one product for q, k and v together (the reference concatenates the three matrices and
their biases at load time too, qwen_infer.c:1316-1367), rotation of q and k fused with the append
of k and v to the pages, attention of every row over the pages of its own request, and the output
product.  All rows' keys and values are in the cache before any row's attention runs
(qwen_infer.c:2017-2023), which is what makes a prompt portion causal.

Options of the spec, each off for the plain form: values of another size than keys; an RMS norm of the whole query
row and of the whole key row of a token before the rotation, or of every head by itself; a softmax whose denominator is
enlarged by one, or by exp of a learned number per head; scores squashed by c tanh(s / c); queries that see the keys of their
own block of positions only; a gate, sigmoid of a further
product of the mixer's input, on the joined heads before the output product, feature by feature or one number per head.  The gate's matrix is
one more block of rows of the one q/k/v product.  With any of the first two the kernel that norms, rotates and appends
is `qk_norm_rope_append`.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np
import torch

from ..csrc import ops
from .cache_need import PagedKVNeed, PagedKVView
from .context import BuildContext
from .linear import Linear
from .registry import register_mixer
from .rope import shared_position
from .spec import AttentionSpec, TensorRole
from .stream import ResidualStream


@register_mixer("gqa_attention")
class GQAAttention:
    @staticmethod
    def expected_tensors(spec: AttentionSpec) -> List[TensorRole]:
        qd, kvd = spec.n_heads * spec.head_dim, spec.n_kv_heads * spec.head_dim
        vvd, od = spec.n_kv_heads * spec.value_dim, spec.n_heads * spec.value_dim
        roles = [TensorRole("q_proj.weight", (qd, spec.hidden), True, True),
                 TensorRole("o_proj.weight", (spec.hidden, od), True, True)]
        if spec.own_kv:
            roles += [TensorRole("k_proj.weight", (kvd, spec.hidden), True, True),
                      TensorRole("v_proj.weight", (vvd, spec.hidden), True, True)]
        if spec.qkv_bias:
            roles.append(TensorRole("q_proj.bias", (qd,), role="bias"))
            if spec.own_kv:
                roles += [TensorRole("k_proj.bias", (kvd,), role="bias"), TensorRole("v_proj.bias", (vvd,), role="bias")]
        if spec.out_bias:
            roles.append(TensorRole("o_proj.bias", (spec.hidden,), role="bias"))
        if spec.qk_norm is not None:
            per_head = spec.qk_norm == "head"          # one vector of head_dim weights for all heads of a kind
            roles.append(TensorRole("q_norm.weight", (spec.head_dim if per_head else qd,), role="scale"))
            if spec.own_kv:
                roles.append(TensorRole("k_norm.weight", (spec.head_dim if per_head else kvd,), role="scale"))
        if spec.gate is not None:
            roles.append(TensorRole("g_proj.weight", (spec.n_heads if spec.gate == "head" else od, spec.hidden), True, True))
        if spec.sink == "learned":
            roles.append(TensorRole("sink", (spec.n_heads,)))
        return roles

    cache_need_takes_context = True        # cache_need(spec, ctx): what a page holds depends on the compute type

    @staticmethod
    def stored_head(spec: AttentionSpec, ctx: Optional[BuildContext]) -> Optional[int]:
        """The width at which the heads of an extended attention are stored so that the tensor-core kernels take them (64
        or 128 features, zeros behind a head's own; a zero adds nothing to a score or to a weighted sum), or None where
        they are stored as they are: in float32, for heads that fit already, and where the padding would more than
        double the cache."""
        if ctx is None or ctx.compute_dtype != torch.bfloat16 or ctx.attention == "generic":
            return None
        hd, vd = spec.head_dim, spec.value_dim
        if spec.qk_norm is None and vd == hd and spec.gate is None:
            return None                        # the plain form keeps its layout
        if hd == vd and hd in (64, 128):
            return None
        stored = 64 if max(hd, vd) <= 64 else 128
        return stored if max(hd, vd) <= 128 and stored <= hd + vd else None

    @staticmethod
    def cache_need(spec: AttentionSpec, ctx: Optional[BuildContext] = None) -> Optional[PagedKVNeed]:
        if not spec.own_kv:
            return None
        stored = GQAAttention.stored_head(spec, ctx)
        if stored is not None:
            return PagedKVNeed(spec.n_kv_heads, stored, spec.window, None, spec.block)
        return PagedKVNeed(spec.n_kv_heads, spec.head_dim, spec.window,
                           None if spec.value_dim == spec.head_dim else spec.value_dim, spec.block)

    def __init__(self, spec: AttentionSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"{spec.n_heads} query heads are not a multiple of {spec.n_kv_heads} kv heads")
        if spec.head_dim % 2 or spec.head_dim > 256:
            raise ValueError(f"head_dim={spec.head_dim} must be even and at most 256")
        self.spec, self.ctx = spec, ctx
        if spec.qk_norm not in (None, "projection", "head"):
            raise ValueError(f"unknown query/key norm '{spec.qk_norm}' (projection, head)")
        if spec.gate not in (None, "elementwise", "head"):
            raise ValueError(f"unknown output gate '{spec.gate}' (elementwise, head)")
        if spec.sink not in (False, True, "learned"):
            raise ValueError(f"unknown sink '{spec.sink}' (False, True, learned)")
        if spec.score_cap is not None and not spec.score_cap > 0.0:
            raise ValueError(f"score_cap={spec.score_cap} must be positive")
        self.nh, self.nkv, self.hd, self.vd = spec.n_heads, spec.n_kv_heads, spec.head_dim, spec.value_dim
        if self.vd <= 0 or self.vd > 256:
            raise ValueError(f"v_head_dim={self.vd} must be positive and at most 256")
        self.qd, self.kvd = self.nh * self.hd, self.nkv * self.hd
        self.od = self.nh * self.vd
        # what the plain form does not have: the step between product and attention is then a kernel of its own
        self.extended = spec.qk_norm is not None or self.vd != self.hd or spec.gate is not None
        if self.extended and not spec.own_kv:
            raise ValueError("the extended attention has a cache of its own")
        names = ["q_proj"] + (["k_proj", "v_proj"] if spec.own_kv else [])
        w = torch.cat([tensors[n + ".weight"] for n in names] + ([tensors["g_proj.weight"]] if spec.gate else []), dim=0)
        b = torch.cat([tensors[n + ".bias"].float() for n in names], dim=0) if spec.qkv_bias else None
        if b is not None and spec.gate:                # the gate's rows of the one product have no bias
            b = torch.cat([b, torch.zeros(tensors["g_proj.weight"].shape[0], dtype=b.dtype, device=b.device)])
        self.gate_col = self.qd + (self.kvd + self.nkv * self.vd if spec.own_kv else 0)
        pad = (-w.shape[0]) % 8
        if spec.gate == "head" and pad:                # one gate per head: rows of zeros behind them keep the product's
            w = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=w.dtype, device=w.device)], dim=0)       # rows 16 bytes apart
            if b is not None:
                b = torch.cat([b, torch.zeros(pad, dtype=b.dtype, device=b.device)])
        f32 = lambda t: t.to(device=ctx.device, dtype=torch.float32).contiguous()
        self.q_norm = f32(tensors["q_norm.weight"]) if spec.qk_norm else None
        self.k_norm = f32(tensors["k_norm.weight"]) if spec.qk_norm else None
        self.sink_weight = f32(tensors["sink"]) if spec.sink == "learned" else None
        self.score_cap = float(np.float32(spec.score_cap)) if spec.score_cap is not None else 0.0
        self.qkv = Linear(w, b, ctx, label="proj_qkv")
        self.o_proj = Linear(tensors["o_proj.weight"], tensors.get("o_proj.bias") if spec.out_bias else None, ctx,
                             label="proj_o")
        self.position = shared_position(spec.position, ctx)
        scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(float(self.hd))
        self.scale = float(np.float32(scale))
        # (a softmax with the enlarged denominator runs the kernels that have it)
        self.stored = self.stored_head(spec, ctx)
        khd, kvd_ = (self.hd, self.vd) if self.stored is None else (self.stored, self.stored)     # what the kernels see
        self.plans = {d: ops.attention_plan(self.nh // self.nkv, khd, ctx.cache_dtype, d, ctx.attention,
                                            ctx.page_size, vd=kvd_, softcap=self.score_cap > 0.0,
                                            learned_sink=self.sink_weight is not None) for d in (False, True)}
        if spec.block is not None and (spec.window is not None or spec.block <= 0):
            raise ValueError("blocks of positions stand in place of a window and hold at least one position")
        # what the kernels are told: a positive number is a sliding window, a negative one the size of the blocks
        self.window = int(spec.window) if spec.window else (-int(spec.block) if spec.block else 0)
        # the fused q/k/v product can rotate and append itself: whole heads rotated in halves, a cache of its own
        # in bfloat16
        self.rope_in_product = (spec.own_kv and self.position.rotary_dim == self.hd and not self.position.interleaved
                                and ctx.compute_dtype == torch.bfloat16 and ctx.cache_dtype == torch.bfloat16
                                and not self.extended)

    takes_stream = True        # forward takes a NormedInput and may add its result to the stream itself

    def forward(self, h, batch, cache: PagedKVView, stream: Optional[ResidualStream] = None) -> Optional[torch.Tensor]:
        """h: the normed rows, or a NormedInput.  With `stream` the result is added to it (or left owed to
        it) and None is returned; without, the addend is returned."""
        T = batch.n_rows
        qkv = None
        khd, kvd_ = (self.hd, self.vd) if self.stored is None else (self.stored, self.stored)
        if self.extended:
            qkv = self.qkv.of(h)
            q = torch.empty((T, self.nh * khd), dtype=self.ctx.compute_dtype, device=qkv.device)
            ops.qk_norm_rope_append(qkv, q, T, self.nh, self.nkv, self.hd, self.vd, self.position.rotary_dim,
                                    self.position.interleaved, self.q_norm, self.k_norm, self.spec.qk_norm_eps,
                                    self.position.table(batch), batch.positions, batch.row_req, cache.block_table,
                                    cache.pool, cache.page_size, self.ctx.status, stored=self.stored,
                                    per_head=self.spec.qk_norm == "head")
        elif self.rope_in_product and self.qkv.rope_fuses(T, self.hd):
            # a step of few tokens: rotation and cache append inside the q/k/v product
            q = torch.empty((T, self.qd), dtype=self.ctx.compute_dtype, device=self.ctx.device)
            self.qkv.of_rope(h, q, (self.position.table(batch), batch.positions, batch.row_req, cache.block_table,
                                    cache.pool, cache.page_size, self.nh, self.nkv, self.hd))
        else:
            qkv = self.qkv.of(h)
            q = torch.empty((T, self.qd), dtype=self.ctx.compute_dtype, device=qkv.device)
            ops.rope_kv_append(qkv, q, T, self.nh, self.nkv, self.hd, self.position.rotary_dim, self.position.interleaved,
                               self.position.table(batch), batch.positions, batch.row_req, cache.block_table,
                               cache.pool if self.spec.own_kv else None, cache.page_size, self.ctx.status)
        kernel, bq, tile = self.plans[bool(getattr(batch, "decode_only", False))]
        qblk, n_qblk = batch.query_blocks(bq)
        if qblk is None and kernel != "mma_keys":
            batch.implicit_blocks = False              # this kernel wants the list
            qblk, n_qblk = batch.query_blocks(bq)
        out = torch.empty((T, self.nh * kvd_), dtype=self.ctx.compute_dtype, device=q.device)
        ops.attention(q, q.stride(0), cache.pool, cache.block_table, batch.positions, qblk, n_qblk,
                      batch.max_position, T, self.nh, self.nkv, khd, self.window, self.ctx.kv_split, tile, bq,
                      self.scale, out, self.ctx.status, kernel, vd=kvd_, sink=bool(self.spec.sink),
                      sink_weight=self.sink_weight, softcap=self.score_cap)
        gate_per = self.vd if self.spec.gate == "head" else 1      # one gate per head, or one per feature
        if self.spec.gate is not None and self.stored is None:
            ops.sigmoid_gate(out, qkv, self.gate_col, self.od, gate_per=gate_per)
        elif self.spec.gate is not None:               # the gate's kernel also drops the zeros behind every head
            wide, out = out, torch.empty((T, self.od), dtype=self.ctx.compute_dtype, device=q.device)
            ops.sigmoid_gate(out, qkv, self.gate_col, self.od, src=wide, vd=self.vd, head_stride=self.stored, gate_per=gate_per)
        elif self.stored is not None:
            out = out.view(T, self.nh, self.stored)[:, :, :self.vd].reshape(T, self.od)
        if stream is None:
            return self.o_proj.partial(out)
        self.o_proj.into(out, stream)
        return None
