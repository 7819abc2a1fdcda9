"""A decoder put together from a `ModelSpec`: embedding, the layers' blocks in the spec's run order,
final norm and head.  The class knows no architecture; which parts run and with which sizes is the
spec's business, and which tensors they get is decided by name.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..csrc import ops
from ..parts import registry
from ..parts.context import BuildContext
from ..parts.linear import Linear
from ..parts.spec import ModelSpec
from ..parts.stream import ResidualStream


class DecoderModel:
    def __init__(self, spec: ModelSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        """`tensors` maps checkpoint names to tensors (any device) in their stored types."""
        import beglin_b200.parts  # noqa: F401
        self.spec, self.ctx = spec, ctx
        if ctx.status is None:
            ctx.status = ops.new_status(ctx.device)
        self.embed = ctx.matrix(tensors[spec.embed_name])
        self.blocks = []
        for layer in spec.layers:
            parts = {}
            for slot, _, cls, pspec in registry.layer_slots(layer):
                mine = {}
                for role in cls.expected_tensors(pspec):
                    name = layer.names[f"{slot}.{role.name}"]
                    if name in tensors:
                        mine[role.name] = tensors[name]
                parts[slot] = cls(pspec, mine, ctx)
            self.blocks.append(registry.block_class(layer.block)(**parts, **getattr(layer, "block_args", {})))
        # parts that stand in front of stages (the input of a pass of a repeated run of layers)
        self.entries = []
        for entry in spec.entries:
            cls = registry.entry_class(entry.part.kind)
            mine = {role.name: tensors[entry.names[role.name]] for role in cls.expected_tensors(entry.part)
                    if entry.names[role.name] in tensors}
            self.entries.append(cls(entry.part, mine, ctx))
        self.keep_origin = any(getattr(e, "needs_origin", False) for e in self.entries)
        self.final_norm = registry.norm_class(spec.final_norm.kind)(
            spec.final_norm, {"weight": tensors[spec.final_norm_name]}, ctx)
        head_bias = None if spec.head_bias_name is None else tensors[spec.head_bias_name]
        if spec.head_name is None:
            self.head = Linear(self.embed, head_bias, ctx, label="head_gemv")     # ctx.matrix is a no-op on the table: one copy
        else:
            self.head = Linear(tensors[spec.head_name], head_bias, ctx, label="head_gemv")

    # ------------------------------------------------------------------ cache
    def cache_needs(self) -> List[Optional[object]]:
        """The cache need of every stage of the run order (None for a stage that reads another's)."""
        needs = []
        for stage in self.spec.order:
            need = None
            if stage.cache is None:
                for _, family, cls, pspec in registry.layer_slots(self.spec.layers[stage.layer]):
                    if family == "mixer":
                        # (a mixer whose pages depend on the compute type is asked with the context)
                        need = cls.cache_need(pspec, self.ctx) if getattr(cls, "cache_need_takes_context", False) \
                            else cls.cache_need(pspec)
            needs.append(need)
        return needs

    def weight_bytes(self) -> int:
        """Bytes of every weight a step reads once (the tied head counted once)."""
        seen, total = set(), 0

        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()

        def walk(obj, depth=0):
            if isinstance(obj, torch.Tensor):
                add(obj)
            elif isinstance(obj, (list, tuple)):
                for v in obj:
                    walk(v, depth)
            elif depth < 3 and hasattr(obj, "__dict__"):
                for k, v in vars(obj).items():
                    if k in ("ctx", "spec", "bias_c", "embed"):
                        continue
                    walk(v, depth + 1)

        for b in self.blocks:
            for part in vars(b).values():
                walk(part)
        for e in self.entries:
            walk(e)
        walk(self.final_norm)
        walk(self.head)
        return total

    # ------------------------------------------------------------------ forward
    def forward(self, batch, cache, tap=None) -> Optional[torch.Tensor]:
        """Run the batch's rows through every stage, from and into `cache`; return float logits
        [wanted rows, vocab], or None when no row's logits are wanted (the head is skipped then, as
        qwen_infer.c:2145 skips it).  `tap(stage, rows)` is called behind every stage with a copy of the
        float residual stream [T, hidden] as that stage leaves it (for looking into a model layer by layer; it
        reads what the stream still owes, so it is not for captured steps)."""
        x = torch.empty((batch.n_rows, self.spec.hidden), dtype=torch.float32, device=self.ctx.device)
        ops.embed_gather(self.embed, batch.token_ids, x, self.ctx.status, scale=self.spec.embed_scale)
        stream = ResidualStream(x)
        if self.keep_origin:
            stream.origin = x.clone()
        if self.spec.lanes:
            stream.open_lanes(self.spec.lanes)
        for si, stage in enumerate(self.spec.order):
            if stage.enter is not None:
                self.entries[stage.enter].forward(stream, batch)
            owner = si if stage.cache is None else stage.cache
            view = cache.view(owner, batch) if owner in cache.stage_group else None
            self.blocks[stage.layer].forward(stream, batch, view)
            if tap is not None and stream.lanes is not None:
                lanes = stream.lanes.clone()
                if stream.lane_owed is not None:
                    y, link = stream.lane_owed
                    y = y.float().reshape(-1, *lanes.shape[1:]).sum(0)
                    lanes = torch.einsum("ab,atd->btd", link.mix, lanes) + link.out[:, None, None] * y
                tap(si, lanes.sum(0))
            elif tap is not None:
                rows = stream.x.clone()
                if stream.pending is not None:
                    rows += stream.pending.float().reshape(-1, *rows.shape).sum(0)
                if stream.terms is not None:
                    for t, c in stream.terms.items:
                        rows += c * t.float().reshape(-1, *rows.shape).sum(0)
                tap(si, rows)
        if batch.n_logit_rows == 0:
            return None
        if stream.lanes is not None:               # the final norm reads the sum of the lanes, at the wanted rows
            h = self.final_norm.add_norm(stream.lane_sum(batch.logit_rows), None, update=False)
        else:
            stream.settle()
            h = self.final_norm.add_norm(stream.x, stream.pending, rows=batch.logit_rows, update=False)
        logits = self.head(h, out_dtype=torch.float32)
        if self.spec.logit_softcap > 0.0:
            ops.softcap(logits, self.spec.logit_softcap)
        return logits
