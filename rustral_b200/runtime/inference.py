"""InferencePool: a bounded queue in front of worker threads (crates/runtime/src/inference.rs:22-76).
`infer` blocks for the reply; a full queue applies back-pressure to callers."""
from __future__ import annotations

import queue
import threading


class PoolClosed(RuntimeError):
    pass


class InferenceResponse:
    """What a worker hands back (crates/runtime/src/inference.rs:16-19): `output`, or `error` when the handler raised."""

    __slots__ = ("output", "error")

    def __init__(self, output=None, error: BaseException | None = None):
        self.output, self.error = output, error

    def unwrap(self):
        if self.error is not None:
            raise self.error
        return self.output


class InferenceRequest:
    """One queued call (crates/runtime/src/inference.rs:7-13): the input and the reply slot the worker fills.
    `InferencePool.submit` returns it; `wait()` blocks for the `InferenceResponse`."""

    __slots__ = ("input", "_box", "_ev")

    def __init__(self, inp):
        self.input, self._box, self._ev = inp, [], threading.Event()

    def wait(self, timeout: float | None = None) -> InferenceResponse:
        if not self._ev.wait(timeout):
            raise TimeoutError("inference timed out")
        ok, val = self._box[0]
        return InferenceResponse(val) if ok else InferenceResponse(error=val)

    def done(self) -> bool:
        return self._ev.is_set()


class InferencePool:
    def __init__(self, workers: int, queue_bound: int, handler):
        self._q: queue.Queue = queue.Queue(maxsize=max(1, queue_bound))
        self._handler = handler
        self._closed = False
        self._threads = [threading.Thread(target=self._run, daemon=True) for _ in range(max(1, workers))]
        for t in self._threads:
            t.start()

    def _run(self):
        while True:
            item = self._q.get()
            if item is None:
                return
            inp, box, ev = item
            try:
                box.append((True, self._handler(inp)))
            except BaseException as e:   # noqa: BLE001 - delivered to the caller
                box.append((False, e))
            ev.set()

    def submit(self, inp, timeout: float | None = None) -> InferenceRequest:
        """Queues `inp` and returns at once; several requests can be in flight from one caller."""
        if self._closed:
            raise PoolClosed("pool is shut down")
        req = InferenceRequest(inp)
        self._q.put((inp, req._box, req._ev), timeout=timeout)
        return req

    def infer(self, inp, timeout: float | None = None):
        return self.submit(inp, timeout).wait(timeout).unwrap()

    def shutdown(self):
        if self._closed:
            return
        self._closed = True
        for _ in self._threads:
            self._q.put(None)
        for t in self._threads:
            t.join(timeout=5)
