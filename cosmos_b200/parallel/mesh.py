"""Device mesh over (dp_replicate, dp_shard, cfgp, cp, tp) with one process group per axis.

Rank layout (slowest to fastest): dp_replicate, dp_shard, cfgp, cp, tp. Keeping cp and tp
innermost puts the chattiest groups on consecutive ranks; on an NVSwitch box every pair of
GPUs has the same bandwidth, so this only matters for readability of the layout.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch.distributed as dist

from ..config import ParallelConfig

AXES = ("dp_replicate", "dp_shard", "cfgp", "cp", "tp")


class Mesh:
    def __init__(self, pc: ParallelConfig, world: int, rank: int, create_groups: bool = True):
        pc.validate(world)
        self.pc, self.world, self.rank = pc, world, rank
        self.sizes = {a: getattr(pc, a) for a in AXES}
        self.coords = self.coords_of(rank)
        self.groups: Dict[str, Optional[dist.ProcessGroup]] = {a: None for a in AXES}
        self.group_ranks: Dict[str, List[int]] = {a: self.ranks_along(a, rank) for a in AXES}
        if create_groups and world > 1 and dist.is_initialized():
            for a in AXES:
                if self.sizes[a] == 1:
                    continue
                # every rank must create every group, in the same order
                seen = set()
                for r in range(world):
                    members = tuple(self.ranks_along(a, r))
                    if members in seen:
                        continue
                    seen.add(members)
                    g = dist.new_group(list(members))
                    if rank in members:
                        self.groups[a] = g

    def coords_of(self, rank: int) -> Dict[str, int]:
        out, r = {}, rank
        for a in reversed(AXES):
            out[a] = r % self.sizes[a]
            r //= self.sizes[a]
        return out

    def rank_of(self, coords: Dict[str, int]) -> int:
        r = 0
        for a in AXES:
            r = r * self.sizes[a] + coords[a]
        return r

    def ranks_along(self, axis: str, rank: int) -> List[int]:
        c = self.coords_of(rank)
        return [self.rank_of({**c, axis: i}) for i in range(self.sizes[axis])]

    def size(self, axis: str) -> int:
        return self.sizes[axis]

    def index(self, axis: str) -> int:
        return self.coords[axis]

    def group(self, axis: str):
        return self.groups[axis]

    def describe(self) -> str:
        parts = [f"{a}{self.sizes[a]}" for a in AXES if self.sizes[a] > 1]
        s = "x".join(parts) if parts else "single"
        if self.sizes["cp"] > 1:
            s += f"({self.pc.cp_mode})"
        return s
