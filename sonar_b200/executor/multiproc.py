"""One worker process per GPU, driven from the engine-core process.

The executor spawns ``world_size`` processes, each of which joins the
``torch.distributed`` job, builds its ``Worker`` and then serves RPCs in a busy
loop.  Calls are broadcast through one shared-memory ring (every worker sees
every call); replies come back over one ring per worker — all workers answer
``collective_rpc``, only the output rank answers ``execute_model``.  A monitor
thread watches the process sentinels: a worker that dies marks the executor
failed, wakes any pending call with ``WorkerDeadError`` and invokes the failure
callback (the engine reports itself dead to its clients).

Parity: ``aphrodite/v1/executor/multiproc_executor.py:103`` (``collective_rpc`` :337,
monitor :267, ``WorkerProc`` :539, ``worker_busy_loop`` :947).
"""
from __future__ import annotations

import multiprocessing as mp
import os
from collections import deque
import signal
import socket
import threading
import time
import traceback
from multiprocessing.connection import wait as mp_wait
from typing import Any

from sonar_b200 import envs
from sonar_b200.config import EngineConfig
from sonar_b200.executor.base import Executor
from sonar_b200.executor.shm_queue import MessageQueue, QueueHandle, QueueTimeout
from sonar_b200.logger import init_logger

logger = init_logger(__name__)


class WorkerDeadError(RuntimeError):
    pass


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker_main(cfg: EngineConfig, rank: int, world: int, init_method: str, rpc: QueueHandle, resp: QueueHandle,
                 ready, parent_pid: int) -> None:
    signal.signal(signal.SIGINT, signal.SIG_IGN)
    from sonar_b200.worker.worker import Worker
    rpc_q = MessageQueue.attach(rpc, rank)
    resp_q = MessageQueue.attach(resp, None)
    try:
        worker = Worker(cfg, rank=rank, local_rank=rank, world_size=world, init_method=init_method)
        worker.init_device()
        worker.load_model()
        ready.set()
    except Exception:
        resp_q.put(("error", traceback.format_exc()))
        raise
    # Steps launched with defer=True whose sampled tokens have not been read back yet, oldest first.  The
    # engine runs at most one step ahead: the reply to step N goes out once step N+1 has been launched (or
    # when the engine asks with "__resolve__", or before any other call is served, so replies keep call order).
    pending: deque = deque()

    def finish(item) -> None:
        deferred, reply_ranks = item
        try:
            out, status = deferred.result(), "ok"
        except Exception:
            out, status = traceback.format_exc(), "error"
        if reply_ranks is None or rank in reply_ranks or status == "error":
            resp_q.put((status, out))

    while True:
        try:
            msg = rpc_q.get(timeout_s=2.0)
        except QueueTimeout:
            if os.getppid() != parent_pid:      # the engine is gone: do not linger
                return
            continue
        method, args, kwargs, reply_ranks = msg
        if method == "__shutdown__":
            worker.shutdown()
            return
        if method == "execute_model" and kwargs.get("defer"):
            try:
                pending.append((worker.execute_model(*args, defer=True), reply_ranks))
            except Exception:
                while pending:
                    finish(pending.popleft())
                resp_q.put(("error", traceback.format_exc()))
                continue
            while len(pending) > 1:
                finish(pending.popleft())
            continue
        while pending:
            finish(pending.popleft())
        if method == "__resolve__":
            continue
        try:
            out = getattr(worker, method)(*args, **kwargs)
            status = "ok"
        except Exception:
            out, status = traceback.format_exc(), "error"
        if reply_ranks is None or rank in reply_ranks or status == "error":
            resp_q.put((status, out))


class _MPDeferred:
    """The reply to a step launched ahead; ``result()`` reads it (and the ones before it) off the reply queue."""

    def __init__(self, executor: "MultiprocExecutor") -> None:
        self.executor, self.done, self.value = executor, False, None

    def result(self):
        return self.executor._resolve(self)


class MultiprocExecutor(Executor):
    @property
    def supports_defer(self) -> bool:          # run-ahead needs the sampled tokens on the rank that launches
        return self.cfg.parallel.pipeline_parallel_size == 1

    def execute_model(self, so, defer: bool = False):
        if not defer or not self.supports_defer:
            return self.collective_rpc("execute_model", so, output_rank_only=True)[0]
        if self.is_failed:
            raise WorkerDeadError("a worker process has died")
        with self._lock:
            self.rpc_q.put(("execute_model", (so,), {"defer": True}, [self.output_rank]),
                           timeout_s=envs.SONAR_RPC_TIMEOUT_S)
            d = _MPDeferred(self)
            self._deferred.append(d)
        return d

    def _read_reply(self, rank: int, what: str, timeout_s: float):
        deadline = time.time() + timeout_s
        while True:
            if self.is_failed:
                raise WorkerDeadError("a worker process has died")
            try:
                status, val = self.resp_qs[rank].get(timeout_s=0.5)
                break
            except QueueTimeout:
                if time.time() > deadline:
                    raise TimeoutError(f"worker {rank} did not answer {what} within {timeout_s}s") from None
        if status != "ok":
            raise RuntimeError(f"worker {rank} failed in {what}:\n{val}")
        return val

    def _resolve(self, d: _MPDeferred):
        with self._lock:
            return self._resolve_locked(d)

    def _resolve_locked(self, d: _MPDeferred | None):
        """Read deferred replies in launch order up to ``d`` (all of them for ``None``).  The workers answer
        step N by themselves once step N+1 is launched; the newest step needs the explicit flush."""
        while self._deferred and (d is None or not d.done):
            if len(self._deferred) == 1:
                self.rpc_q.put(("__resolve__", (), {}, None), timeout_s=envs.SONAR_RPC_TIMEOUT_S)
            oldest = self._deferred[0]
            try:
                oldest.value = self._read_reply(self.output_rank, "execute_model", envs.SONAR_RPC_TIMEOUT_S)
            finally:
                oldest.done = True
                self._deferred.pop(0)
        return d.value if d is not None else None

    def _init_executor(self) -> None:
        cfg = self.cfg
        self._deferred: list[_MPDeferred] = []
        self.world = cfg.parallel.world_size
        ctx = mp.get_context("spawn")
        self.rpc_q = MessageQueue.create(self.world, slot_bytes=1 << 20, n_slots=8)
        self.resp_qs = [MessageQueue.create(1, slot_bytes=1 << 20, n_slots=4) for _ in range(self.world)]
        for q in self.resp_qs:
            q.reader = 0
        init_method = f"tcp://127.0.0.1:{_free_port()}"
        self.procs = []
        readies = []
        for r in range(self.world):
            ev = ctx.Event()
            p = ctx.Process(target=_worker_main, name=f"sonar-worker-{r}",
                            args=(cfg, r, self.world, init_method, self.rpc_q.handle, self.resp_qs[r].handle, ev,
                                  os.getpid()), daemon=True)
            p.start()
            self.procs.append(p)
            readies.append(ev)
        deadline = time.time() + envs.SONAR_RPC_TIMEOUT_S
        for r, ev in enumerate(readies):
            while not ev.wait(timeout=0.5):
                if not self.procs[r].is_alive():
                    self.shutdown()
                    raise WorkerDeadError(f"worker {r} exited during start-up (code {self.procs[r].exitcode})")
                if time.time() > deadline:
                    self.shutdown()
                    raise TimeoutError(f"worker {r} did not start within {envs.SONAR_RPC_TIMEOUT_S}s")
        # the last pipeline stage's first TP rank holds the sampled tokens
        p = cfg.parallel
        self.output_rank = (p.pipeline_parallel_size - 1) * p.tensor_parallel_size * p.prefill_context_parallel_size
        self._closing = False
        self._lock = threading.Lock()
        self._monitor = threading.Thread(target=self._watch, daemon=True)
        self._monitor.start()

    def _watch(self) -> None:
        sentinels = [p.sentinel for p in self.procs]
        dead = mp_wait(sentinels)
        if self._closing:
            return
        self.is_failed = True
        idx = [i for i, p in enumerate(self.procs) if p.sentinel in dead]
        logger.error("worker process(es) %s died unexpectedly", idx)
        if self._failure_cb is not None:
            self._failure_cb()

    def collective_rpc(self, method: str, *args, output_rank_only: bool = False, timeout_s: float | None = None,
                       **kwargs) -> list[Any]:
        if self.is_failed:
            raise WorkerDeadError("a worker process has died")
        timeout_s = timeout_s or envs.SONAR_RPC_TIMEOUT_S
        ranks = [self.output_rank] if output_rank_only else list(range(self.world))
        with self._lock:
            self._resolve_locked(None)          # replies of steps still in flight come first
            self.rpc_q.put((method, args, kwargs, ranks if output_rank_only else None), timeout_s=timeout_s)
            out = []
            deadline = time.time() + timeout_s
            for r in ranks:
                while True:
                    if self.is_failed:
                        raise WorkerDeadError("a worker process has died")
                    try:
                        status, val = self.resp_qs[r].get(timeout_s=0.5)
                        break
                    except QueueTimeout:
                        if time.time() > deadline:
                            raise TimeoutError(f"worker {r} did not answer {method} within {timeout_s}s") from None
                if status != "ok":
                    raise RuntimeError(f"worker {r} failed in {method}:\n{val}")
                out.append(val)
            return out

    def shutdown(self) -> None:
        if getattr(self, "_closing", False):
            return
        self._closing = True
        try:
            if not self.is_failed:
                self.rpc_q.put(("__shutdown__", (), {}, None), timeout_s=2.0)
        except Exception:  # noqa: BLE001
            pass
        for p in getattr(self, "procs", []):
            p.join(timeout=5)
            if p.is_alive():
                p.terminate()
        for q in [getattr(self, "rpc_q", None), *getattr(self, "resp_qs", [])]:
            if q is not None:
                q.close()
