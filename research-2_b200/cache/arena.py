"""The memory that the cache manager's indices point into.

Per cache group one tensor [num_pages + 1, page_elems]: page 0 is the null page (real memory,
never handed out). A page holds, for each member layer of the group, K then V for `page_size`
tokens, each laid out [kv_head][offset][head_dim] (values with a head size of their own where a
layer has one; no V at all for a member whose values lie inside its key rows), so a (page, head) tile is contiguous. One
block table per request and group therefore serves all the group's layers (the reference packs
all layers of a group into one page row too: kelpie-models/kelpie_models/sdk/kv.py:1-34,
118-143). Per-request state of fixed size lives beside it: one tensor [max_requests, *shape]
per state-holding mixer, indexed by the request's state slot.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .manager import GroupSpec


@dataclass(frozen=True)
class MemberSpec:
    """What one layer's cache needs: a group (by window and kept first tokens) and the sizes of a
    token's K and V (`v_head_dim` 0: values have the keys' head size). `values_in_keys`: a token's value is the first
    v_head_dim numbers of its key row (a cache of latents): the pages hold key rows only."""

    n_kv_heads: int
    head_dim: int
    window: int = 0
    v_head_dim: int = 0
    keep_first: int = 0
    values_in_keys: bool = False

    @property
    def value_dim(self) -> int:
        return self.v_head_dim or self.head_dim

    @property
    def stored_value_dim(self) -> int:
        return 0 if self.values_in_keys else self.value_dim

    @property
    def lifetime(self) -> tuple[int, int]:
        """Members whose pages live equally long: without a window every position is kept anyway."""
        return (self.window, self.keep_first if self.window > 0 else 0)


@dataclass
class CacheMember:
    """One layer's K and V inside its group's pages (pointers + strides for the kernels)."""

    group: int
    k: torch.Tensor  # 1-D views into the group's tensor; only their data_ptr is used
    v: torch.Tensor
    page_stride: int  # elements between consecutive pages
    page_size: int
    n_pages: int  # including the null page
    n_kv_heads: int
    head_dim: int
    window: int
    v_head_dim: int = 0  # 0: the keys' head size
    keep_first: int = 0


def derive_groups(members: list[MemberSpec], page_size: int, num_pages: int) -> tuple[list[GroupSpec], list[int]]:
    """Members with the same lifetime (here: the same window and the same kept first tokens) share a group
    (kelpie-models/kelpie_models/sdk/groups.py:268-294). -> (groups, group index per member)."""
    keys: list[tuple[int, int]] = []
    index: list[int] = []
    for m in members:
        if m.lifetime not in keys:
            keys.append(m.lifetime)
        index.append(keys.index(m.lifetime))
    if not keys:  # a model without any per-token cache still gets one (empty) group
        keys.append((0, 0))
    return [GroupSpec(page_size, w, num_pages, keep) for w, keep in keys], index


class KVArena:
    def __init__(self, members: list[MemberSpec], groups: list[GroupSpec], member_group: list[int],
                 dtype: torch.dtype, device: torch.device | str):
        self.groups = groups
        self.dtype = dtype
        sizes = [0] * len(groups)
        offsets = []
        for m, g in zip(members, member_group):
            k_elems = m.n_kv_heads * groups[g].page_size * m.head_dim
            v_elems = m.n_kv_heads * groups[g].page_size * m.stored_value_dim
            offsets.append((sizes[g], sizes[g] + k_elems))
            sizes[g] += k_elems + v_elems
        self.tensors = [
            torch.zeros(groups[g].num_pages + 1, max(sizes[g], 1), dtype=dtype, device=device)
            for g in range(len(groups))
        ]
        self.members: list[CacheMember] = []
        for (k_off, v_off), m, g in zip(offsets, members, member_group):
            flat = self.tensors[g].view(-1)
            self.members.append(CacheMember(
                group=g, k=flat[k_off:], v=flat[k_off if m.values_in_keys else v_off:], page_stride=sizes[g], page_size=groups[g].page_size,
                n_pages=groups[g].num_pages + 1, n_kv_heads=m.n_kv_heads, head_dim=m.head_dim, window=m.window,
                v_head_dim=m.v_head_dim, keep_first=m.keep_first,
            ))

    def fill_(self, value: float) -> None:
        """Tests fill the pool with a loud value so that a read of a slot never written shows."""
        for t in self.tensors:
            t.fill_(value)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors)
