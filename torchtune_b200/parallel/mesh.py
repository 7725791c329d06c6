"""Parallel dimensions and process groups (parity: torchtune/training/_distributed.py:61-176)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch.distributed as dist


@dataclass
class ParallelDims:
    """``dp_replicate · dp_shard · cp · tp (· ep shares the dp ranks) == world_size``;
    ``dp_shard = -1`` is inferred."""

    dp_replicate: int = 1
    dp_shard: int = -1
    tp: int = 1
    cp: int = 1
    world_size: int = 1
    ep: int = 1

    def __post_init__(self) -> None:
        self._validate()

    def _validate(self) -> None:
        for name in ("dp_replicate", "tp", "cp", "ep"):
            if getattr(self, name) < 1:
                raise AssertionError(f"{name} must be >= 1")
        if not (self.dp_shard == -1 or self.dp_shard >= 1):
            raise AssertionError("dp_shard must be -1 or >= 1")
        if self.dp_shard < 0:
            denom = self.dp_replicate * self.cp * self.tp
            if self.world_size % denom:
                raise AssertionError(f"world_size {self.world_size} is not divisible by dp_replicate*cp*tp = {denom}")
            self.dp_shard = self.world_size // denom
        if self.dp_replicate * self.dp_shard * self.cp * self.tp != self.world_size:
            raise AssertionError(
                f"Invalid parallel dims: dp_replicate({self.dp_replicate}) * dp_shard({self.dp_shard}) * cp({self.cp}) * tp({self.tp}) != WORLD_SIZE({self.world_size})"
            )
        if (self.dp_replicate * self.dp_shard) % self.ep:
            raise AssertionError("ep must divide the data-parallel size")

    # derived ------------------------------------------------------------
    @property
    def dp_enabled(self) -> bool:
        return self.dp_replicate > 1 or self.dp_shard > 1

    @property
    def dp_replicate_enabled(self) -> bool:
        return self.dp_replicate > 1

    @property
    def dp_shard_enabled(self) -> bool:
        return self.dp_shard > 1

    @property
    def tp_enabled(self) -> bool:
        return self.tp > 1

    @property
    def cp_enabled(self) -> bool:
        return self.cp > 1

    @property
    def dp_size(self) -> int:
        return self.dp_replicate * self.dp_shard

    @property
    def non_data_parallel_size(self) -> int:
        return self.cp * self.tp

    @property
    def min_seq_len_divisor(self) -> int:
        """Sequences are padded to a multiple of this: ``tp`` for sequence parallelism, ``2·tp·cp``
        with load-balanced context parallelism."""
        return self.tp * (self.cp * 2 if self.cp_enabled else 1)

    # rank layout: [dp_replicate, dp_shard, cp, tp] with tp fastest --------------------------
    def coordinates(self, rank: int) -> Dict[str, int]:
        tp = rank % self.tp
        cp = (rank // self.tp) % self.cp
        ds = (rank // (self.tp * self.cp)) % self.dp_shard
        dr = rank // (self.tp * self.cp * self.dp_shard)
        return {"dp_replicate": dr, "dp_shard": ds, "cp": cp, "tp": tp, "dp": dr * self.dp_shard + ds}

    def groups_along(self, dim: str) -> List[List[int]]:
        """Rank lists of every process group along ``dim`` (``dp`` = replicate×shard flattened)."""
        buckets: Dict[Tuple, List[int]] = {}
        for r in range(self.world_size):
            c = self.coordinates(r)
            if dim == "dp":
                key = (c["cp"], c["tp"])
            elif dim == "dp_shard_cp":
                key = (c["dp_replicate"], c["tp"])
            else:
                key = tuple(v for k, v in c.items() if k not in (dim, "dp"))
            buckets.setdefault(key, []).append(r)
        return list(buckets.values())

    def build_groups(self, dims=("dp", "tp", "cp")) -> Dict[str, Optional[dist.ProcessGroup]]:
        """Create the process groups (every rank must call this with the same arguments)."""
        me = dist.get_rank()
        out: Dict[str, Optional[dist.ProcessGroup]] = {}
        for dim in dims:
            mine = None
            for ranks in self.groups_along(dim):
                g = dist.new_group(ranks) if len(ranks) > 1 else None
                if me in ranks:
                    mine = g
            out[dim] = mine
        return out
