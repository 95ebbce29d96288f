"""Device arrays behind the cache manager's pages and state slots.

Per cache number (a run item's `cache`): K and V arrays [pages, kv_heads, page_size, head_dim]
(V with its own width where a mixer asks for one) in the engine's storage dtype (the reference's layout, src/memory/page_atten.zig:2,
src/backend/cuda/attention/attention.cu:12), and/or one state array [slots, *shape].  Cache
numbers that share a group share its page ids; each keeps its own arrays.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import KVRequest, LayerCache, StateRequest
from .manager import FULL, WINDOW, CacheError, GroupSpec


def group_of(req: KVRequest) -> GroupSpec:
    return GroupSpec(req.group_kind, req.window if req.group_kind == WINDOW else 0)


def plan_groups(kv_requests: Dict[int, KVRequest]) -> Tuple[List[GroupSpec], Dict[int, int]]:
    """Distinct groups in order of first use, and each cache number's group index."""
    groups: List[GroupSpec] = []
    index: Dict[int, int] = {}
    for cache_id in sorted(kv_requests):
        g = group_of(kv_requests[cache_id])
        if g not in groups:
            groups.append(g)
        index[cache_id] = groups.index(g)
    if not groups:
        groups.append(GroupSpec(FULL))   # a model without paged state still has one (empty) group
    return groups, index


def bytes_per_page(kv_requests: Dict[int, KVRequest], group_index: Dict[int, int], group: int, page_size: int,
                   dtype: torch.dtype) -> int:
    """Bytes one page id of `group` occupies over all cache numbers of that group."""
    elem = torch.empty((), dtype=dtype).element_size()
    return sum(r.num_kv_heads * page_size * (r.head_dim + r.value_dim) * elem
               for c, r in kv_requests.items() if group_index[c] == group)


class CacheStorage:
    def __init__(self, kv_requests: Dict[int, KVRequest], state_requests: Dict[int, StateRequest],
                 group_index: Dict[int, int], pages_per_group: Sequence[int], page_size: int,
                 num_state_slots: int, dtype: torch.dtype, device):
        self.page_size = page_size
        self.group_index = group_index
        self.kv: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self.state: Dict[int, torch.Tensor] = {}
        for c, r in kv_requests.items():
            shape = (pages_per_group[group_index[c]], r.num_kv_heads, page_size)
            self.kv[c] = (torch.zeros(shape + (r.head_dim,), dtype=dtype, device=device),
                          torch.zeros(shape + (r.value_dim,), dtype=dtype, device=device))
        for c, r in state_requests.items():
            self.state[c] = torch.zeros((num_state_slots, *r.shape), dtype=r.dtype, device=device)

    def layer_cache(self, cache_id: Optional[int], writes: bool) -> LayerCache:
        if cache_id is None:
            return LayerCache(page_size=self.page_size, writes=writes)
        k, v = self.kv.get(cache_id, (None, None))
        return LayerCache(k=k, v=v, group=self.group_index.get(cache_id, 0), page_size=self.page_size,
                          writes=writes, state=self.state.get(cache_id))

    def reset_state(self, slots: Sequence[int]) -> None:
        """Zero the state of slots that were just handed to new requests."""
        if not slots or not self.state:
            return
        for t in self.state.values():
            idx = torch.as_tensor(list(slots), dtype=torch.long, device=t.device)
            t.index_fill_(0, idx, 0)

    def bytes_held(self) -> int:
        n = sum(k.numel() * k.element_size() + v.numel() * v.element_size() for k, v in self.kv.values())
        return n + sum(t.numel() * t.element_size() for t in self.state.values())
