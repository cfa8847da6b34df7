"""EngineHandle: the thread that owns an LLMEngine and the command channel in front of it.

Clients (HTTP handlers, the CLI) never touch the engine directly: they post Enqueue / Cancel /
Shutdown commands and receive TokenEvents on a per-request queue, from any thread or from an
asyncio loop. The worker thread drains commands, runs `engine.step()` while there is work and
idles with a three-phase back-off (spin -> yield -> timed park).

Reference parity: EngineCommand{Enqueue,Cancel,Shutdown} / EngineHandle::generate_stream
(oxide-engine/src/continuous_batching.rs:22-46,1503-1572), ExecutionWorker idle policy spin<=200,
yield<=2000, park 50us (oxide-core/src/worker.rs:90-138), per-request failure isolation
(continuous_batching.rs:664-672,1223-1235,802-804).
"""
from __future__ import annotations

import asyncio
import queue
import threading
import time
from dataclasses import dataclass
from typing import Optional

from ..errors import EngineError, SlotsExhausted
from ..sampling_params import SamplingParams


@dataclass
class StreamEvent:
    req_id: int
    token: int
    finished: bool
    reason: str


class RequestStream:
    """Receives the events of one request; usable from threads (get) and asyncio (aget)."""

    def __init__(self, req_id: int, loop: Optional[asyncio.AbstractEventLoop] = None):
        self.req_id = req_id
        self.loop = loop
        self.q: "queue.Queue[StreamEvent]" = queue.Queue()
        self.aq: Optional[asyncio.Queue] = asyncio.Queue() if loop is not None else None
        self.prompt_tokens = 0
        self.closed = False

    def push(self, ev: StreamEvent) -> None:
        if self.loop is not None and self.aq is not None:
            try:
                self.loop.call_soon_threadsafe(self.aq.put_nowait, ev)
            except RuntimeError:
                self.closed = True  # the client's loop is gone
        else:
            self.q.put(ev)

    def get(self, timeout: Optional[float] = None) -> StreamEvent:
        return self.q.get(timeout=timeout)

    async def aget(self) -> StreamEvent:
        return await self.aq.get()


class EngineHandle:
    def __init__(self, engine, max_slots: Optional[int] = None, native_worker: Optional[bool] = None):
        self.engine = engine
        # With `native_worker` the steps run on the C++ StepWorker (csrc/host/worker.*): a dedicated
        # host thread fed through a single-producer / single-consumer ring of 64-byte commands, with the
        # spin -> yield -> park idle policy and an optional core pin, as in the reference's
        # scheduler-actor / GPU-worker split (continuous_batching.rs:1413-1499, worker.rs:90-138). This
        # thread then only drains commands and hands out step tickets.
        if native_worker is None:
            native_worker = bool(getattr(engine.cfg, "native_worker", False))
        self.native_worker = native_worker
        self._worker = None
        self._worker_error: Optional[str] = None
        self.max_slots = max_slots or engine.cfg.max_num_seqs
        self.cmd: "queue.Queue" = queue.Queue()
        self.streams: dict[int, RequestStream] = {}
        self._ids = 0
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self.healthy = True
        self.last_error: Optional[str] = None
        self.last_step_time = time.monotonic()
        self.thread = threading.Thread(target=self._run, name="oxb-engine-worker", daemon=True)
        self.thread.start()

    # ------------------------------------------------------------------ client side
    def active_slots(self) -> int:
        return len(self.streams)

    def submit(self, prompt_tokens, params: SamplingParams, loop=None, queue_if_full: bool = True) -> RequestStream:
        with self._lock:
            if not queue_if_full and len(self.streams) >= self.max_slots:
                raise SlotsExhausted("All inference slots busy (concurrency limit reached)")
            rid = self._ids
            self._ids += 1
            st = RequestStream(rid, loop)
            st.prompt_tokens = len(prompt_tokens)
            self.streams[rid] = st
        self.cmd.put(("enqueue", rid, list(prompt_tokens), params))
        return st

    def cancel(self, req_id: int) -> None:
        self.cmd.put(("cancel", req_id))

    def shutdown(self, timeout: float = 10.0) -> None:
        self.cmd.put(("shutdown",))
        self._stop.set()
        self.thread.join(timeout)

    def generate(self, prompt_tokens, params: SamplingParams, timeout: float = 600.0):
        """Blocking helper: returns (tokens, finish_reason)."""
        st = self.submit(prompt_tokens, params)
        out = []
        while True:
            ev = st.get(timeout=timeout)
            if ev.token >= 0:
                out.append(ev.token)
            if ev.finished:
                return out, ev.reason

    # ------------------------------------------------------------------ worker side
    def _on_token(self, state, e) -> None:
        st = self.streams.get(int(e.req_id))
        if st is None:
            return
        if st.closed:  # client went away: free the slot
            self.engine.cancel(int(e.req_id))
            self.streams.pop(int(e.req_id), None)
            return
        st.push(StreamEvent(int(e.req_id), int(e.token), bool(e.finished), str(e.reason)))
        if e.finished:
            self.streams.pop(int(e.req_id), None)

    def _drain(self) -> bool:
        got = False
        while True:
            try:
                c = self.cmd.get_nowait()
            except queue.Empty:
                return got
            got = True
            if c[0] == "enqueue":
                _, rid, toks, params = c
                try:
                    self.engine.add_request(toks, params, on_token=self._on_token, req_id=rid)
                except Exception as ex:  # admission failure fails this request only
                    st = self.streams.pop(rid, None)
                    if st is not None:
                        st.push(StreamEvent(rid, -1, True, f"prefill_error: {ex}"))
            elif c[0] == "cancel":
                self.engine.cancel(c[1])
            elif c[0] == "shutdown":
                self._stop.set()
                return got

    def _bind_device(self) -> None:
        """The current CUDA device is per thread: the worker adopts the engine's (a process may hold
        several engines on different GPUs, e.g. data-parallel replicas)."""
        dev = getattr(self.engine, "device", None)
        if dev is not None and getattr(dev, "type", "cpu") == "cuda":
            import torch

            torch.cuda.set_device(dev)

    def _step_on_worker(self, kind: int, a0: int, a1: int):
        """Handler of the native worker thread: one engine step per command."""
        try:
            if not getattr(self, "_worker_bound", False):
                self._bind_device()
                self._worker_bound = True
            self.engine.step()
            return 0, 0
        except EngineError as ex:
            self._worker_error = str(ex)
        except Exception as ex:
            self._worker_error = f"{type(ex).__name__}: {ex}"
        return 1, 0

    def _step(self) -> None:
        """One engine step, on this thread or through the native worker; raises what the step raised."""
        if not self.native_worker:
            self.engine.step()
            return
        if self._worker is None:
            from .._build import host_ext

            pin = int(getattr(self.engine.cfg, "worker_pin_core", -1))
            self._worker = host_ext().StepWorker(self._step_on_worker, capacity=8, pin_core=pin)
            self._tickets = 0
        self._tickets += 1
        while not self._worker.submit(self._tickets):
            time.sleep(0)
        deadline_ms = int(max(1.0, getattr(self.engine.cfg, "step_deadline_s", 30.0)) * 1000)
        done = self._worker.wait(deadline_ms)
        if done is None:
            raise EngineError(f"step worker did not finish a step within {deadline_ms} ms")
        if done[1] != 0:
            msg, self._worker_error = self._worker_error or "step failed on the worker thread", None
            raise EngineError(msg)

    def _run(self) -> None:
        self._bind_device()
        idle = 0
        while not self._stop.is_set():
            busy = self._drain()
            if self.engine.has_work():
                try:
                    self._step()
                    self.last_step_time = time.monotonic()
                    self.healthy = not self.engine.stats.get("degraded", False)
                except EngineError as ex:
                    self._fail_all(str(ex))
                except Exception as ex:  # keep the server alive, fail the in-flight requests
                    self._fail_all(f"{type(ex).__name__}: {ex}")
                idle = 0
                continue
            if busy:
                idle = 0
                continue
            idle += 1
            if idle <= 200:
                continue
            if idle <= 2000:
                time.sleep(0)
            else:
                time.sleep(50e-6 if idle < 20000 else 1e-3)
        if self._worker is not None:
            self._worker.stop()
            self._worker = None
        for rid, st in list(self.streams.items()):
            st.push(StreamEvent(rid, -1, True, "cancelled"))
        self.streams.clear()

    def _fail_all(self, msg: str) -> None:
        self.healthy = False
        self.last_error = msg
        for rid in list(self.streams.keys()):
            try:
                self.engine.cancel(rid)
            except Exception:
                pass
            st = self.streams.pop(rid, None)
            if st is not None:
                st.push(StreamEvent(rid, -1, True, f"prefill_error: {msg}"))
        self.healthy = True  # the engine itself is still usable for new requests
