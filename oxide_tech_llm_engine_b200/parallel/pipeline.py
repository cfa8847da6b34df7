"""Pipeline parallelism: contiguous layer ranges per stage, hidden-state hand-off over
`torch.distributed` point-to-point (NCCL send/recv on GPUs, gloo on CPU ranks), micro-batched so
that a stage computes micro-batch i+1 while its send of micro-batch i is in flight.

The scheduler is replicated on every stage (same requests, same decisions); the last stage samples
and broadcasts the token ids so that every replica applies the same update.

Reference parity: `layer_partition_for_gpu` (remainder-aware split, oxide-backend-cuda/src/nccl.rs:
110-120), the `-ngl` layer planner WeightAllocator::plan (oxide-models/src/loader.rs:118-158) and
the "1F1B" note of oxide-engine/src/distributed.rs:5; the reference moves no data between devices.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist

from .mesh import layer_partition_for_rank


@dataclass(frozen=True)
class StagePlan:
    pp: int
    stage: int
    n_layers: int

    @property
    def layers(self) -> tuple[int, int]:
        return layer_partition_for_rank(self.n_layers, self.pp, self.stage)

    @property
    def first(self) -> bool:
        return self.stage == 0

    @property
    def last(self) -> bool:
        return self.stage == self.pp - 1


def plan_n_gpu_layers(n_layers: int, n_gpu_layers: int) -> tuple[range, range]:
    """`-ngl N`: the last N layers (and the head) live on the device, the rest on the host."""
    n = n_layers if n_gpu_layers < 0 else min(n_gpu_layers, n_layers)
    return range(0, n_layers - n), range(n_layers - n, n_layers)


class PipelineComm:
    """Point-to-point hand-off between neighbouring stages of one pipeline."""

    def __init__(self, prev_rank: Optional[int], next_rank: Optional[int], group=None):
        self.prev, self.next, self.group = prev_rank, next_rank, group
        self._pending: list = []

    def send(self, x: torch.Tensor) -> None:
        if self.next is not None:
            self._pending.append(dist.isend(x.contiguous(), self.next, group=self.group))

    def recv(self, buf: torch.Tensor):
        if self.prev is None:
            return None
        return dist.irecv(buf, self.prev, group=self.group)

    def flush(self) -> None:
        for w in self._pending:
            w.wait()
        self._pending.clear()


def run_stage_microbatched(plan: StagePlan, comm: PipelineComm, micro_inputs: Sequence,
                           first_fn: Callable, mid_fn: Callable, hidden_like: Callable) -> list:
    """Runs one engine step through this stage for every micro-batch.

    first_fn(mb) -> hidden (stage 0 embeds and runs its layers); mid_fn(mb, hidden) -> hidden or,
    on the last stage, the step's result; hidden_like(mb) allocates the receive buffer. Receives
    for micro-batch i+1 are posted before computing micro-batch i, sends are asynchronous."""
    outs = []
    n = len(micro_inputs)
    bufs = [None if plan.first else hidden_like(mb) for mb in micro_inputs]
    reqs = [None] * n
    if not plan.first and n > 0:
        reqs[0] = comm.recv(bufs[0])
    for i, mb in enumerate(micro_inputs):
        if not plan.first and i + 1 < n:
            reqs[i + 1] = comm.recv(bufs[i + 1])
        if plan.first:
            h = first_fn(mb)
        else:
            reqs[i].wait()
            h = mid_fn(mb, bufs[i])
        if plan.last:
            outs.append(h)
        else:
            comm.send(h)
    comm.flush()
    return outs


def broadcast_tokens(tokens: torch.Tensor, src: int, group=None) -> torch.Tensor:
    """The last stage's sampled ids reach every replica of the scheduler."""
    dist.broadcast(tokens, src, group=group)
    return tokens


@dataclass
class PpContext:
    """Where one rank sits in a (pp x tp) grid: global rank = stage * tp + tp_rank."""
    pp: int
    tp: int
    stage: int
    tp_rank: int
    tp_group: object = None       # ranks of this stage (the fused TP kernels' peers)
    column_group: object = None   # the ranks with the same tp_rank in every stage
    column_src: int = 0           # global rank of the last stage in this column (token source)

    @property
    def first(self) -> bool:
        return self.stage == 0

    @property
    def last(self) -> bool:
        return self.stage == self.pp - 1

    @property
    def prev_rank(self) -> int:
        return (self.stage - 1) * self.tp + self.tp_rank

    @property
    def next_rank(self) -> int:
        return (self.stage + 1) * self.tp + self.tp_rank

    def layers(self, n_layers: int) -> tuple[int, int]:
        return layer_partition_for_rank(n_layers, self.pp, self.stage)


def build_pp_context(rank: int, world: int, pp: int) -> PpContext:
    """Creates the process groups of a pp x tp grid. Every rank of the job must call this (group
    creation is collective), after `init_process_group`."""
    if world % pp:
        raise ValueError(f"world {world} is not a multiple of pp {pp}")
    tp = world // pp
    stage, tp_rank = divmod(rank, tp)
    tp_group = column_group = None
    for st in range(pp):
        g = dist.new_group(list(range(st * tp, (st + 1) * tp)))
        if st == stage:
            tp_group = g
    for c in range(tp):
        g = dist.new_group([st * tp + c for st in range(pp)])
        if c == tp_rank:
            column_group = g
    return PpContext(pp=pp, tp=tp, stage=stage, tp_rank=tp_rank, tp_group=tp_group, column_group=column_group,
                     column_src=(pp - 1) * tp + tp_rank)
