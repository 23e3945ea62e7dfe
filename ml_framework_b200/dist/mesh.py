"""N-dimensional device mesh over ranks.

Same rules as the reference's ``DeviceMesh`` (src/MLFramework/Distributed/Mesh/DeviceMesh.cs:44-205):
ranks are laid out row-major over ``shape`` (last dimension fastest); dimensions are named
Data = 0, Tensor = 1, Pipeline = 2, Expert = 3 (ParallelismDimension.cs:6-26); the group of a
rank along dimension d is the set of ranks that agree with it on every other coordinate;
``tp_group_ranks`` = ranks sharing my Data coordinate (and all others but Tensor),
``dp_group_ranks`` = ranks sharing my Tensor coordinate.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple


class ParallelismDimension(enum.IntEnum):
    DATA = 0
    TENSOR = 1
    PIPELINE = 2
    EXPERT = 3


@dataclass(frozen=True)
class DeviceMeshCoord:
    coords: Tuple[int, ...]

    def __getitem__(self, i: int) -> int:
        return self.coords[i]

    def __len__(self):
        return len(self.coords)


class DeviceMesh:
    def __init__(self, shape: Sequence[int], rank: int, dim_names: Optional[Sequence[str]] = None):
        shape = tuple(int(s) for s in shape)
        if not shape or any(s <= 0 for s in shape):
            raise ValueError(f"mesh shape must be positive, got {shape}")
        self.shape = shape
        self.size = 1
        for s in shape:
            self.size *= s
        if not (0 <= rank < self.size):
            raise ValueError(f"rank {rank} outside mesh of {self.size} ranks")
        self.rank = rank
        self.dim_names = tuple(dim_names) if dim_names else tuple(
            ParallelismDimension(i).name.lower() if i < 4 else f"dim{i}" for i in range(len(shape)))
        self.coord = self.rank_to_coord(rank)
        self._group_cache: Dict[Tuple[int, Tuple[int, ...]], List[int]] = {}
        self._pgs: Dict[int, object] = {}

    @classmethod
    def create_from_rank(cls, rank: int, shape: Sequence[int], dim_names=None) -> "DeviceMesh":
        return cls(shape, rank, dim_names)

    def rank_to_coord(self, rank: int) -> DeviceMeshCoord:
        if not (0 <= rank < self.size):
            raise ValueError("rank out of range")
        c = []
        for s in reversed(self.shape):
            c.append(rank % s)
            rank //= s
        return DeviceMeshCoord(tuple(reversed(c)))

    def coord_to_rank(self, coord) -> int:
        coords = tuple(coord.coords if isinstance(coord, DeviceMeshCoord) else coord)
        if len(coords) != len(self.shape):
            raise ValueError("coordinate rank mismatch")
        r = 0
        for c, s in zip(coords, self.shape):
            if not (0 <= c < s):
                raise ValueError(f"coordinate {coords} outside mesh {self.shape}")
            r = r * s + c
        return r

    def _dim(self, dim) -> int:
        if isinstance(dim, str):
            return self.dim_names.index(dim)
        return int(dim)

    def group_ranks(self, dim, rank: Optional[int] = None) -> List[int]:
        """Ranks that differ from ``rank`` (default: mine) only in coordinate ``dim``."""
        d = self._dim(dim)
        base = self.rank_to_coord(self.rank if rank is None else rank).coords
        key = (d, base[:d] + base[d + 1:])
        if key not in self._group_cache:
            self._group_cache[key] = [self.coord_to_rank(base[:d] + (i,) + base[d + 1:]) for i in range(self.shape[d])]
        return self._group_cache[key]

    def ranks_with_index(self, dim, index: int) -> List[int]:
        """All ranks whose coordinate along ``dim`` equals ``index`` (GetGroupRanks(dim, index))."""
        d = self._dim(dim)
        return [r for r in range(self.size) if self.rank_to_coord(r)[d] == index]

    def all_groups(self, dim) -> List[List[int]]:
        seen, out = set(), []
        for r in range(self.size):
            g = tuple(self.group_ranks(dim, r))
            if g not in seen:
                seen.add(g)
                out.append(list(g))
        return out

    def tp_group_ranks(self) -> List[int]:
        return self.group_ranks(ParallelismDimension.TENSOR) if len(self.shape) > 1 else [self.rank]

    def dp_group_ranks(self) -> List[int]:
        return self.group_ranks(ParallelismDimension.DATA)

    def pp_group_ranks(self) -> List[int]:
        return self.group_ranks(ParallelismDimension.PIPELINE) if len(self.shape) > 2 else [self.rank]

    def local_rank(self, dim) -> int:
        return self.coord[self._dim(dim)]

    def dim_size(self, dim) -> int:
        return self.shape[self._dim(dim)]

    @property
    def tp_world_size(self) -> int:
        return self.shape[1] if len(self.shape) > 1 else 1

    @property
    def dp_world_size(self) -> int:
        return self.shape[0]

    @property
    def pp_world_size(self) -> int:
        return self.shape[2] if len(self.shape) > 2 else 1

    @property
    def tp_rank(self) -> int:
        return self.coord[1] if len(self.shape) > 1 else 0

    @property
    def dp_rank(self) -> int:
        return self.coord[0]

    @property
    def pp_rank(self) -> int:
        return self.coord[2] if len(self.shape) > 2 else 0

    def is_master(self) -> bool:
        return self.rank == 0

    def execute_on_master(self, fn: Callable, *a, **k):
        return fn(*a, **k) if self.is_master() else None

    def process_group(self, dim):
        """The communicator along ``dim`` containing this rank. Every rank of the default group
        must call this for the same ``dim`` (sub-group creation is collective)."""
        from .process_group import new_group
        d = self._dim(dim)
        if d not in self._pgs:
            mine = None
            for g in self.all_groups(d):
                pg = new_group(g)
                if self.rank in g:
                    mine = pg
            self._pgs[d] = mine
        return self._pgs[d]


def init_device_mesh(shape: Sequence[int], dim_names=None) -> DeviceMesh:
    from .process_group import default_group
    pg = default_group()
    mesh = DeviceMesh(shape, pg.rank, dim_names)
    if mesh.size != pg.world_size:
        raise ValueError(f"mesh {tuple(shape)} needs {mesh.size} ranks, world has {pg.world_size}")
    return mesh
