"""
Batch-parallel replicas: one process per GPU, a full copy of the weights in each, no collective in the data path.

The reference scales a DiT across GPUs by giving every process its own images; the only host-side coordination is a
common start, a common end and the sum of the per-process throughputs.  This module is that coordination with failure
reporting: a replica that raises (or dies) is named in the report, the other replicas finish their own work, and no
survivor ever waits on the failed one longer than ``timeout`` seconds.  Nothing here touches a GPU; the worker function
does.

    report = run_replicas(worker, world=8, args=(cfg,))
    report.results      # {rank: value returned by worker(rank, world, sync, *args)}
    report.failed       # {rank: "ExceptionType: message" | "exit code N"}

``sync`` (a :class:`ReplicaSync`) gives the worker ``start()`` (wait until every live replica is ready), ``failed_ranks()``
(cheap check between steps) and ``finish()``.
"""

from __future__ import annotations

import os
import socket
import time
import traceback
from dataclasses import dataclass, field
from datetime import timedelta

import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class ReplicaSync:
    """Start / finish rendezvous over a TCPStore that tolerates missing ranks (no barrier that a dead rank can hang)."""

    def __init__(self, rank: int, world: int, port: int, timeout: float):
        self.rank, self.world, self.timeout = rank, world, timeout
        self.store = dist.TCPStore("127.0.0.1", port, world_size=None, is_master=False,
                                   timeout=timedelta(seconds=timeout), wait_for_workers=False)

    def failed_ranks(self) -> list[int]:
        return [r for r in range(self.world) if self.store.check([f"failed/{r}"])]

    def _rendezvous(self, name: str) -> list[int]:
        """Wait until every rank has either arrived at `name` or been reported failed; returns the failed ranks."""
        self.store.set(f"{name}/{self.rank}", b"1")
        deadline = time.monotonic() + self.timeout
        while True:
            missing = [r for r in range(self.world)
                       if not self.store.check([f"{name}/{r}"]) and not self.store.check([f"failed/{r}"])]
            if not missing:
                return self.failed_ranks()
            if time.monotonic() > deadline:
                for r in missing:  # a rank that never shows up counts as failed; say so for everyone
                    self.store.set(f"failed/{r}", f"no sign of life at '{name}' after {self.timeout:.0f} s".encode())
                return self.failed_ranks()
            time.sleep(0.01)

    def start(self) -> list[int]:
        return self._rendezvous("start")

    def finish(self) -> list[int]:
        return self._rendezvous("finish")

    def report_failure(self, message: str) -> None:
        self.store.set(f"failed/{self.rank}", message.encode())


@dataclass
class ReplicaReport:
    world: int
    results: dict = field(default_factory=dict)
    failed: dict = field(default_factory=dict)

    @property
    def ok(self) -> bool:
        return not self.failed and len(self.results) == self.world

    def raise_for_failures(self) -> None:
        if self.failed:
            names = ", ".join(f"rank {r} ({why})" for r, why in sorted(self.failed.items()))
            raise ReplicaFailure(f"{len(self.failed)} of {self.world} replicas failed: {names}", self)


class ReplicaFailure(RuntimeError):
    def __init__(self, msg: str, report: ReplicaReport):
        super().__init__(msg)
        self.report = report


def _child(rank, world, port, timeout, worker, args, queue, visible_devices):
    if visible_devices is not None:
        os.environ["CUDA_VISIBLE_DEVICES"] = str(visible_devices[rank])  # before the worker initialises CUDA
    sync = None
    try:
        sync = ReplicaSync(rank, world, port, timeout)
        queue.put((rank, "ok", worker(rank, world, sync, *args)))
    except BaseException as e:  # the report must name this rank whatever went wrong
        why = f"{type(e).__name__}: {e}"
        try:
            if sync is not None:
                sync.report_failure(why)
        finally:
            queue.put((rank, "error", why + "\n" + traceback.format_exc(limit=4)))
        raise SystemExit(1)


def run_replicas(worker, world: int, args: tuple = (), timeout: float = 60.0, visible_devices=None,
                 join_timeout: float | None = None) -> ReplicaReport:
    """
    Run ``worker(rank, world, sync, *args)`` in ``world`` spawned processes and collect a :class:`ReplicaReport`.
    ``visible_devices[rank]`` (optional) becomes the child's ``CUDA_VISIBLE_DEVICES``.  A child that raises is reported
    under its rank with the exception text; one that disappears without a message is reported with its exit code.
    """
    ctx = mp.get_context("spawn")
    port = _free_port()
    store = dist.TCPStore("127.0.0.1", port, world_size=None, is_master=True, timeout=timedelta(seconds=timeout),
                          wait_for_workers=False)
    queue = ctx.Queue()
    procs = [ctx.Process(target=_child, args=(r, world, port, timeout, worker, args, queue, visible_devices))
             for r in range(world)]
    for p in procs:
        p.start()
    report = ReplicaReport(world)
    deadline = time.monotonic() + (join_timeout if join_timeout is not None else 10 * timeout)
    pending = set(range(world))
    while pending and time.monotonic() < deadline:
        try:
            rank, kind, payload = queue.get(timeout=0.2)
        except Exception:
            for r in list(pending):  # a child that died without a word (killed, segfault)
                if procs[r].exitcode is not None and procs[r].exitcode != 0:
                    time.sleep(0.2)
                    if queue.empty():
                        report.failed[r] = f"exit code {procs[r].exitcode}"
                        store.set(f"failed/{r}", report.failed[r].encode())
                        pending.discard(r)
            continue
        pending.discard(rank)
        if kind == "ok":
            report.results[rank] = payload
        else:
            report.failed[rank] = payload.splitlines()[0]
    for r in pending:
        report.failed[r] = "no result before the launcher's deadline"
    for p in procs:
        p.join(timeout=5)
        if p.is_alive():
            p.terminate()
    del store
    return report
