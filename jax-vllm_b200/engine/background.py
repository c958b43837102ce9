"""Delivery of a driver's events to the callers that wait for them, with or without a background thread.

Every request that is added gets a queue of its own.  `events(request_id)` yields the request's events until
the one that finishes it.  With the background thread running, the thread steps the engine and hands every
step's events to the queues; readers sleep on one condition variable and are woken by the delivery (nobody
polls, and an idle thread sleeps on the same condition until a request arrives).  Without a thread, the reader
steps the engine itself and the events of other requests wait in their queues.

An exception inside the thread is kept (`failure`): the thread ends, every reader and every later call of the
entry point raises it again, as the reference's engine does with its own loop (jllm/engine/engine.py:230-233).
"""

from __future__ import annotations

import threading
import traceback
from collections import deque
from typing import Callable, Iterator, Optional


class EngineFailed(RuntimeError):
    """The background thread died; the text names the exception that killed it."""


class EventRouter:
    def __init__(self, step: Callable[[], list], has_work: Callable[[], bool]):
        self._step, self._has_work = step, has_work
        self._cv = threading.Condition()
        self._queues: dict[int, deque] = {}
        self._thread: Optional[threading.Thread] = None
        self._stopping = False
        self._was_started = False
        self.failure: Optional[str] = None

    # --------------------------------------------------------------------- queues
    def open(self, request_id: int) -> None:
        with self._cv:
            self._queues[request_id] = deque()

    def close(self, request_id: int) -> None:
        with self._cv:
            self._queues.pop(request_id, None)

    def deliver(self, events) -> None:
        if not events:
            return
        with self._cv:
            for ev in events:
                q = self._queues.get(ev.request_id)
                if q is not None:
                    q.append(ev)
            self._cv.notify_all()

    def wake(self) -> None:
        """There is new work (a request was added): an idle thread looks again."""
        with self._cv:
            self._cv.notify_all()

    # --------------------------------------------------------------------- thread
    @property
    def running(self) -> bool:
        return self._thread is not None and self._thread.is_alive()

    def raise_if_failed(self) -> None:
        if self.failure is not None:
            raise EngineFailed(f"the engine's background thread died of {self.failure}")

    def start(self) -> None:
        if self.running:
            return
        with self._cv:
            self.failure, self._stopping, self._was_started = None, False, True
        self._thread = threading.Thread(target=self._loop, name="jax-vllm-b200-engine", daemon=True)
        self._thread.start()

    def stop(self, join: bool = True) -> None:
        with self._cv:
            self._stopping = True
            self._cv.notify_all()
        if join and self._thread is not None:
            self._thread.join()
            self._thread = None

    def _loop(self) -> None:
        try:
            while True:
                with self._cv:
                    self._cv.wait_for(lambda: self._stopping or self._has_work())
                    if self._stopping:
                        return
                self.deliver(self._step())
        except BaseException as exc:      # kept for every reader and every later call
            traceback.print_exc()
            with self._cv:
                self.failure = f"{type(exc).__name__}: {exc}"
                self._stopping = True
                self._cv.notify_all()

    # -------------------------------------------------------------------- readers
    def events(self, request_id: int) -> Iterator:
        with self._cv:
            q = self._queues.get(request_id)
        if q is None:
            raise KeyError(f"request {request_id} has no events to read: it was never added, or they were read to the end")
        while True:
            with self._cv:
                self._cv.wait_for(lambda: q or self.failure is not None or not self.running)
                ev = q.popleft() if q else None
                failed, threaded = self.failure is not None, self._was_started
            if ev is None:
                if failed:
                    self.raise_if_failed()
                if threaded:
                    raise RuntimeError(f"the engine was stopped with request {request_id} unfinished")
                # no thread was ever started: this reader drives the engine
                produced = self._step()
                if not produced and not self._has_work():
                    raise RuntimeError(f"the engine has no work left, yet request {request_id} is unfinished")
                self.deliver(produced)
                continue
            yield ev
            if ev.finished:
                self.close(request_id)
                return
