"""Parallel mesh coordinates, tensor-split planning and pipeline layer partitioning.

Reference parity: ParallelMeshConfig / MeshCoordinate::from_global_rank with the order
tp -> cp -> ep -> dp -> pp (oxide-engine/src/distributed.rs:14-80), TpColumnLinear
(distributed.rs:84-107), RingAttentionStep peers (distributed.rs:109-142), the proportional
slice planner TensorSplitMode (tensor_split.rs:11-160) and layer_partition_for_gpu
(oxide-backend-cuda/src/nccl.rs:110-120). In the reference these are descriptors only; here
they drive the real sharding of `models.llama.DeviceModel`.
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum


@dataclass(frozen=True)
class ParallelMeshConfig:
    tp: int = 1
    pp: int = 1
    dp: int = 1
    ep: int = 1
    cp: int = 1

    @property
    def world_size(self) -> int:
        return self.tp * self.cp * self.ep * self.dp * self.pp

    def validate(self) -> None:
        for k in ("tp", "pp", "dp", "ep", "cp"):
            if getattr(self, k) < 1:
                raise ValueError(f"{k} must be >= 1")


@dataclass(frozen=True)
class MeshCoordinate:
    tp: int
    cp: int
    ep: int
    dp: int
    pp: int

    @staticmethod
    def from_global_rank(rank: int, mesh: ParallelMeshConfig) -> "MeshCoordinate":
        if not 0 <= rank < mesh.world_size:
            raise ValueError(f"rank {rank} outside a mesh of {mesh.world_size}")
        r = rank
        tp = r % mesh.tp
        r //= mesh.tp
        cp = r % mesh.cp
        r //= mesh.cp
        ep = r % mesh.ep
        r //= mesh.ep
        dp = r % mesh.dp
        r //= mesh.dp
        return MeshCoordinate(tp, cp, ep, dp, r)

    def to_global_rank(self, mesh: ParallelMeshConfig) -> int:
        return (((self.pp * mesh.dp + self.dp) * mesh.ep + self.ep) * mesh.cp + self.cp) * mesh.tp + self.tp


class TensorSplitMode(Enum):
    COLUMN = "column"      # output features sharded (QKV, gate/up, LM head)
    ROW = "row"            # input features sharded (O, down); partial sums are reduce-scattered
    PIPELINE = "pipeline"  # whole layers per rank
    EXPERT = "expert"      # whole experts per rank


def split_sizes(total: int, parts: int, weights: list[float] | None = None, multiple: int = 1) -> list[int]:
    """Proportional split of `total` units into `parts` (remainder to the first ranks)."""
    if weights is None:
        base, rem = divmod(total // multiple, parts)
        return [(base + (1 if i < rem else 0)) * multiple for i in range(parts)]
    s = sum(weights)
    units = total // multiple
    out = [int(units * w / s) for w in weights]
    for i in range(units - sum(out)):
        out[i % parts] += 1
    return [o * multiple for o in out]


def shard_range(total: int, parts: int, idx: int, multiple: int = 1) -> tuple[int, int]:
    sizes = split_sizes(total, parts, multiple=multiple)
    lo = sum(sizes[:idx])
    return lo, lo + sizes[idx]


def layer_partition_for_rank(n_layers: int, pp: int, stage: int) -> tuple[int, int]:
    """Remainder-aware contiguous layer range of one pipeline stage."""
    return shard_range(n_layers, pp, stage)


@dataclass(frozen=True)
class RingAttentionStep:
    chunk_seq_len: int
    send_peer: int
    recv_peer: int

    @staticmethod
    def plan(seq_len: int, cp: int, rank: int) -> "RingAttentionStep":
        return RingAttentionStep((seq_len + cp - 1) // cp, (rank - 1) % cp, (rank + 1) % cp)
