"""One background thread that runs file-writing jobs in submission order (reference: io/background_writer.py:34-111).

The GPU loop hands over host copies of the logits and returns to the next seed while compression and
disk writes proceed; ``close()`` drains the queue and re-raises the first failure.
"""

from __future__ import annotations

import queue
import threading


class BackgroundWriter:
    def __init__(self, max_pending: int = 8):
        self._q: queue.Queue = queue.Queue(maxsize=max_pending)
        self._err: BaseException | None = None
        self._t = threading.Thread(target=self._run, name="df3-writer", daemon=True)
        self._t.start()

    def _run(self):
        while True:
            job = self._q.get()
            try:
                if job is None:
                    return
                fn, args, kwargs = job
                if self._err is None:
                    fn(*args, **kwargs)
            except BaseException as exc:  # noqa: BLE001 - reported by close()
                self._err = exc
            finally:
                self._q.task_done()

    def submit(self, fn, *args, **kwargs) -> None:
        if self._err is not None:
            self.close()
        self._q.put((fn, args, kwargs))

    def close(self) -> None:
        if self._t.is_alive():
            self._q.put(None)
            self._t.join()
        if self._err is not None:
            err, self._err = self._err, None
            raise RuntimeError(f"background write failed: {err!r}") from err

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


def logits_to_host(output):
    """Copy the logit tensors of a ``DeepFold3Output`` to pinned host memory without blocking the stream."""
    import dataclasses

    import torch

    def host(t):
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            return t
        buf = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        buf.copy_(t, non_blocking=True)
        return buf

    out = dataclasses.replace(output, **{f.name: host(getattr(output, f.name)) for f in dataclasses.fields(output)})
    if torch.cuda.is_available():
        torch.cuda.current_stream().synchronize()
    return out
