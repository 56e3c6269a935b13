"""Device storage behind the cache manager's page ids and state slots.

One tensor pair per layer group, laid out ``[layer in group, page, kv head, token in
page, head_dim]``: the ``page_tokens x head_dim`` tile of one head is contiguous, so an
attention kernel streams whole tiles.  (The reference keeps ``(num_blocks, block_size,
H, D)`` per layer, src/minigpt_infer/cache/paged.py:109-123.)  State layers get one
tensor ``[slot, *shape]`` each.  Storage is sized once, from the pool sizes.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .manager import CacheManager


@dataclass
class PagedKVView:
    """What an attention layer sees of the cache in one step."""

    k_pages: torch.Tensor          # [page, kv head, page_tokens, head_dim]
    v_pages: torch.Tensor
    group: int
    page_tokens: int
    window: int | None
    writes: bool


@dataclass
class StateView:
    state: torch.Tensor            # [slot, *shape]
    writes: bool


class CacheStorage:
    def __init__(self, manager: CacheManager, dtype: torch.dtype, device) -> None:
        self.manager = manager
        self.dtype = dtype
        self.device = torch.device(device)
        self.k: list[torch.Tensor] = []
        self.v: list[torch.Tensor] = []
        for group in manager.groups:
            shape = (len(group.layers), group.num_pages, group.spec.n_kv_head,
                     group.page_tokens, group.spec.head_dim)
            self.k.append(torch.zeros(shape, dtype=dtype, device=self.device))
            self.v.append(torch.zeros(shape, dtype=dtype, device=self.device))
        self.state: dict[int, torch.Tensor] = {}
        for layer, spec in manager.state_layers.items():
            self.state[layer] = torch.zeros((manager.max_requests, *spec.shape),
                                            dtype=getattr(torch, spec.dtype), device=self.device)

    def layer_view(self, cache_layer: int, writes: bool = True):
        m = self.manager
        if cache_layer in m.group_of_layer:
            g = m.group_of_layer[cache_layer]
            idx = m.groups[g].layers.index(cache_layer)
            return PagedKVView(self.k[g][idx], self.v[g][idx], g, m.groups[g].page_tokens,
                               m.groups[g].spec.window, writes)
        if cache_layer in self.state:
            return StateView(self.state[cache_layer], writes)
        return None

    def bytes_per_token(self) -> int:
        total = 0
        for g, group in enumerate(self.manager.groups):
            total += (2 * len(group.layers) * group.spec.n_kv_head * group.spec.head_dim
                      * self.k[g].element_size())
        return total
