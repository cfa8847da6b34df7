"""Serving front of a multi-rank engine: rank 0 talks to clients, every rank runs the engine.

A tensor- or expert-parallel engine is one `LLMEngine` per GPU whose schedulers must see the same
request stream in the same order. Rank 0 owns the client-facing side (the HTTP server posts to a
`DistributedEngineHandle`); once per loop iteration it broadcasts the commands that arrived since
the last one (admitted requests with their token ids and sampling parameters, cancellations,
shut-down) to the follower ranks over a host-side **gloo** group, then every rank applies them and
runs the same `engine.step()`. The GPUs never take part in this control traffic; token events are
produced on every rank and delivered to clients by rank 0 only.

Failure handling, all on the host and between steps: every rank beats in the job's key/value
store (`watchdog.Heartbeat`); rank 0 checks the followers before each broadcast
(`watchdog.RankMonitor`) and a follower that left or went silent ends every request with
`rank_failure: ...`, returns all KV blocks and marks the front unhealthy (HTTP 503 from then on).
A failed broadcast (closed socket, group time-out) is treated the same way. When rank 0's own step
raised, it tells the followers to drop their requests and re-arm their hand-off counters too, so
the schedulers stay identical.

Reference surface: `run_server_with_options` -> engine -> router
(oxide-cli/src/lib.rs:1774-1884) and `EngineHandle` / `EngineCommand`
(oxide-engine/src/continuous_batching.rs:22-46,1503-1572); the reference has one process and one
GPU, so the broadcast has no counterpart there.
"""
from __future__ import annotations

import datetime
import queue
import time
from typing import Optional

from ..engine.handle import EngineHandle, StreamEvent
from ..errors import EngineError


def _broadcast(cmds: list, group, src: int = 0) -> list:
    import torch.distributed as dist

    box = [cmds]
    dist.broadcast_object_list(box, src=src, group=group)
    return box[0]


def _drop_everything(engine, reason: str, group) -> None:
    """All ranks together: end every request, and re-arm the hand-off counters only when no rank
    has a kernel in flight any more (a late peer store into a freshly zeroed flag would poison the
    next step), hence the two barriers around the reset."""
    import torch.distributed as dist

    engine.fail_all(reason)
    reset = getattr(getattr(engine, "model", None), "reset_sync_state", None)
    if reset is None:
        return
    import torch

    if torch.cuda.is_available() and not getattr(engine, "cpu", False):
        torch.cuda.synchronize(engine.device)
    dist.barrier(group=group)
    reset()
    dist.barrier(group=group)


def _apply(engine, cmds: list, group=None, on_token=None, on_reject=None) -> bool:
    """Applies one iteration's commands to this rank's engine. Returns True on shut-down."""
    stop = False
    for c in cmds:
        kind = c[0]
        if kind == "enqueue":
            _, rid, toks, params = c
            try:
                engine.add_request(toks, params, on_token=on_token, req_id=rid)
            except Exception as ex:  # the same exception on every rank: the request is refused everywhere
                if on_reject is not None:
                    on_reject(rid, ex)
        elif kind == "cancel":
            engine.cancel(c[1])
        elif kind == "fail_all":
            _drop_everything(engine, c[1], group)
        elif kind == "shutdown":
            stop = True
    return stop


class DistributedEngineHandle(EngineHandle):
    """`EngineHandle` of rank 0 in a multi-rank job (see the module docstring)."""

    def __init__(self, engine, ctl_group, world: int, *, monitor=None, heartbeat=None, store=None,
                 max_slots: Optional[int] = None, idle_beat_s: float = 1.0):
        self.ctl_group = ctl_group
        self.world = world
        self.monitor = monitor
        self.heartbeat = heartbeat
        self.idle_beat_s = idle_beat_s
        self.check_period_s = 0.1          # liveness / fault polling of the job store, off the per-step path
        self._last_check = 0.0
        self._faults_seen: dict = {}
        self.store = store
        self.dead: Optional[str] = None   # set once the group is broken: no further broadcasts
        super().__init__(engine, max_slots)

    def submit(self, prompt_tokens, params, loop=None, queue_if_full: bool = True):
        if self.dead is not None:
            raise EngineError(f"engine group is down: {self.dead}")
        return super().submit(prompt_tokens, params, loop=loop, queue_if_full=queue_if_full)

    def _follower_fault(self) -> Optional[str]:
        """A follower whose step raised (a device wait that ran out on its GPU) dropped its requests
        and says so in the job store (`fault/<rank>` = count:message); rank 0 then makes every rank
        drop and re-arm together."""
        if self.store is None:
            return None
        for r in range(1, self.world):
            key = f"fault/{r}"
            try:
                if not self.store.check([key]):
                    continue
                v = self.store.get(key).decode()
            except Exception:
                continue
            if self._faults_seen.get(r) != v:
                self._faults_seen[r] = v
                return f"rank {r}: {v.split(':', 1)[-1]}"
        return None

    def _collect(self) -> list:
        cmds = []
        while True:
            try:
                c = self.cmd.get_nowait()
            except queue.Empty:
                return cmds
            cmds.append(c)

    def _group_down(self, why: str) -> None:
        self.dead = why
        self.healthy = False
        self.last_error = why
        try:
            self.engine.fail_all(f"rank_failure: {why}")
        except Exception:
            pass
        for rid in list(self.streams.keys()):
            st = self.streams.pop(rid, None)
            if st is not None:
                st.push(StreamEvent(rid, -1, True, f"rank_failure: {why}"))

    def _reject(self, rid: int, ex: Exception) -> None:
        st = self.streams.pop(rid, None)
        if st is not None:
            st.push(StreamEvent(rid, -1, True, f"prefill_error: {ex}"))

    def _run(self) -> None:
        self._bind_device()
        last_beat = time.monotonic()
        pending_fail: Optional[str] = None
        idle = 0
        while not self._stop.is_set():
            if self.dead is not None:
                # the group is gone: answer what still arrives with the failure, never broadcast again
                for c in self._collect():
                    if c[0] == "enqueue":
                        self._reject(c[1], EngineError(self.dead))
                    elif c[0] == "shutdown":
                        self._stop.set()
                time.sleep(1e-3)
                continue
            cmds = self._collect()
            if pending_fail is not None:
                cmds.insert(0, ("fail_all", pending_fail))
                pending_fail = None
            work = self.engine.has_work()
            now = time.monotonic()
            if not cmds and not work:
                if now - last_beat < self.idle_beat_s:
                    idle += 1
                    time.sleep(0 if idle < 2000 else 1e-3)
                    continue
                cmds = [("noop",)]   # keeps the followers' group time-out from running out while idle
            idle = 0
            last_beat = now
            try:
                if now - self._last_check >= self.check_period_s:
                    self._last_check = now
                    if self.monitor is not None:
                        self.monitor.check()
                    fault = self._follower_fault()
                    if fault is not None:
                        self._fail_all(fault)
                        cmds.insert(0, ("fail_all", fault))
                _broadcast(cmds, self.ctl_group)
            except Exception as ex:
                self._group_down(f"{type(ex).__name__}: {ex}")
                continue
            if _apply(self.engine, cmds, self.ctl_group, on_token=self._on_token, on_reject=self._reject):
                self._stop.set()
                break
            if self.engine.has_work():
                try:
                    self.engine.step()
                    self.last_step_time = time.monotonic()
                    self.healthy = not self.engine.stats.get("degraded", False)
                except Exception as ex:
                    msg = str(ex) if isinstance(ex, EngineError) else f"{type(ex).__name__}: {ex}"
                    self._fail_all(msg)
                    pending_fail = msg   # the followers drop their copies with the next broadcast
        if self.dead is None:
            try:
                _broadcast([("shutdown",)], self.ctl_group)
            except Exception:
                pass
        for rid, st in list(self.streams.items()):
            st.push(StreamEvent(rid, -1, True, "cancelled"))
        self.streams.clear()
        if self.heartbeat is not None:
            self.heartbeat.leave()


def follower_loop(engine, ctl_group, *, heartbeat=None, store=None, rank: int = 1,
                  leave_after_steps: Optional[int] = None) -> int:
    """Ranks other than 0: receive each iteration's commands, apply them, run the same step.
    Returns the number of steps run. `leave_after_steps` makes the rank leave the job in an orderly
    way between two steps (the host-side failure tests use it)."""
    steps = faults = 0
    try:
        while True:
            cmds = _broadcast(None, ctl_group)
            if _apply(engine, cmds, ctl_group):
                break
            if engine.has_work():
                try:
                    engine.step()
                except EngineError as ex:
                    # this rank's requests are gone (the engine dropped them); tell rank 0, which makes
                    # every rank drop and re-arm together with its next broadcast
                    faults += 1
                    if store is None:
                        raise
                    store.set(f"fault/{rank}", f"{faults}:{ex}")
                steps += 1
                if leave_after_steps is not None and steps >= leave_after_steps:
                    break
    finally:
        if heartbeat is not None:
            heartbeat.leave()
    return steps


def make_control_group(timeout_s: float = 1800.0):
    """The host-side (gloo) group of all ranks that carries the commands."""
    import torch.distributed as dist

    return dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))


def job_store():
    """The key/value store of the running job (the rendezvous store of torch.distributed)."""
    import torch.distributed as dist

    return dist.distributed_c10d._get_default_store()
