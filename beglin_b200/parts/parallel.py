"""Mixers side by side: every branch reads the same normed input, and the result is the sum of the branches' results,
each times a constant of its own.

The branches are ordinary mixers of the registry (attention, a recurrence, ...), built from their own specs; branch i's
tensors are called `<label i>.<name>`.  Each branch has the cache its kind asks for: the stage's need is the composite
of the branches' needs, and the stage's view is the tuple of their views.  The sum is float: the part hands the block
its branches' results as terms (result, constant), and the kernel that adds a layer's results to the stream adds them
one by one, so the branches' results are never rounded to a sum of their own.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from . import registry
from .cache_need import CompositeNeed
from .context import BuildContext
from .spec import ParallelMixersSpec, TensorRole
from .stream import NormedInput, Terms


@registry.register_mixer("parallel_mixers")
class ParallelMixers:
    @staticmethod
    def _branches(spec: ParallelMixersSpec):
        if not (len(spec.branches) == len(spec.scales) == len(spec.labels)) or not spec.branches:
            raise ValueError("parallel mixers: one constant and one label per branch")
        return [(label, registry.mixer_class(b.kind), b) for label, b in zip(spec.labels, spec.branches)]

    @staticmethod
    def expected_tensors(spec: ParallelMixersSpec) -> List[TensorRole]:
        roles = []
        for label, cls, b in ParallelMixers._branches(spec):
            for r in cls.expected_tensors(b):
                roles.append(TensorRole(f"{label}.{r.name}", r.shape, r.required, r.matrix, r.role))
        return roles

    cache_need_takes_context = True

    @staticmethod
    def cache_need(spec: ParallelMixersSpec, ctx: Optional[BuildContext] = None) -> Optional[CompositeNeed]:
        needs = []
        for _, cls, b in ParallelMixers._branches(spec):
            needs.append(cls.cache_need(b, ctx) if getattr(cls, "cache_need_takes_context", False) else cls.cache_need(b))
        return CompositeNeed(tuple(needs)) if any(n is not None for n in needs) else None

    def __init__(self, spec: ParallelMixersSpec, tensors: Dict[str, torch.Tensor], ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        self.parts = []
        for label, cls, b in self._branches(spec):
            mine = {name[len(label) + 1:]: t for name, t in tensors.items() if name.startswith(label + ".")}
            self.parts.append(cls(b, mine, ctx))
        self.scales = [float(c) for c in spec.scales]

    takes_stream = True
    gives_terms = True         # forward returns Terms: (result, constant) per branch, to be summed in float by the block

    def forward(self, h, batch, cache, stream=None) -> Terms:
        if isinstance(h, NormedInput):
            h = h.tensor()
        views = cache if cache is not None else (None,) * len(self.parts)
        terms = Terms()
        for part, view, scale in zip(self.parts, views, self.scales):
            if getattr(part, "takes_stream", False):
                a = part.forward(h, batch, view, None)
            else:
                a = part.forward(h, batch, view)
            terms.add(a, scale)
        return terms
