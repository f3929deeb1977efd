"""Device memory behind the cache manager: one pool tensor per page group and one
state tensor per stateful layer call.

Pool of a group: ``[entries, pages, 2, kv_heads, page_size, head_dim]`` in the compute
dtype; ``pool[e]`` is what the kernels of cache entry ``e`` index with page numbers
from the block table.  The reference keeps one tensor ``[layers, 2, blocks, block_size,
heads, head_dim]`` (heteroserve/kv/torch_blocks.py:48); here the tile of one (page, head)
is contiguous so that attention can fetch it in one piece.
"""

from __future__ import annotations

import torch


class CacheStorage:
    def __init__(self, model, manager, dtype: torch.dtype, device):
        self.dtype, self.device = dtype, device
        self.page_size = manager.page_size
        self.pools: list[torch.Tensor] = []
        for g, pool in zip(model.cache_groups, manager.pools):
            self.pools.append(torch.zeros(
                (len(g.entries), pool.num_pages, 2, g.kv_heads, manager.page_size, g.head_dim),
                dtype=dtype, device=device))
        self.states: dict[int, torch.Tensor] = {
            idx: torch.zeros((manager.max_requests, *shape), dtype=torch.float32, device=device)
            for idx, shape in model.state_shapes.items()}

    def entry_pool(self, group: int, index: int) -> torch.Tensor:
        return self.pools[group][index]

    def nbytes(self) -> int:
        return (sum(p.numel() * p.element_size() for p in self.pools)
                + sum(s.numel() * 4 for s in self.states.values()))
