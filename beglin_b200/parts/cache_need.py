"""What a mixer asks of the cache manager, and what it is handed back each step.

A mixer's class method `cache_need(spec)` returns one of the needs below (or None).  Stages whose
needs are equal share a group of the cache manager: one page pool and one block table per request
for paged keys and values, one slab of slots for per-request state of fixed size.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values of every position (window None) or of the last `window` positions.  `v_head_dim` is given
    when values have another size than keys.  `block` b: a query reads only the positions of its own block of b positions
    (blocks counted from position 0), so the pages wholly in front of the newest block are given back."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    v_head_dim: Optional[int] = None
    block: Optional[int] = None

    def page_shape(self, page_size: int) -> Tuple[int, ...]:
        """What one page of one stage holds: (2 = keys, values; kv heads; positions; features); with values of
        another size than keys, flat: the keys (kv heads; positions; head_dim) followed by the values (kv heads;
        positions; v_head_dim)."""
        if self.v_head_dim is None or self.v_head_dim == self.head_dim:
            return (2, self.n_kv_heads, page_size, self.head_dim)
        return (self.n_kv_heads * page_size * (self.head_dim + self.v_head_dim),)


@dataclass(frozen=True)
class PagedLatentNeed:
    """ONE row of `width` features per position, shared by all heads (the latent of an attention that makes
    its keys and values from a low-rank projection, with whatever rides along, such as a rotated key part)."""
    width: int
    window: Optional[int] = None
    block: Optional[int] = None

    def page_shape(self, page_size: int) -> Tuple[int, ...]:
        return (page_size, self.width)


PAGED_NEEDS = (PagedKVNeed, PagedLatentNeed)


@dataclass(frozen=True)
class FixedStateNeed:
    """A tensor of this shape per request, zero when the request starts, kept between steps."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


@dataclass(frozen=True)
class CompositeNeed:
    """Several needs of one stage, for a mixer made of branches that keep different things (pages of keys and values beside
    a state of fixed size).  Each joins the group of its own kind; the stage's view is the tuple of their views, with None
    where a branch keeps nothing."""
    needs: Tuple[Optional[object], ...]


@dataclass
class PagedKVView:
    """One stage's pages, [num_pages, 2, n_kv_heads, page_size, head_dim] (2 = keys, values) for keys and values
    or [num_pages, page_size, width] for a latent, and the step's block table [requests, max_pages] (int32, -1
    where no page is held)."""
    pool: torch.Tensor
    block_table: torch.Tensor
    page_size: int
    window: Optional[int]


@dataclass
class FixedStateView:
    """One stage's state slab [slots, *shape] and the step's slot of each request [requests]."""
    state: torch.Tensor
    slots: torch.Tensor
