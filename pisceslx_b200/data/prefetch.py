"""Background batch prefetcher: a host thread pulls batches from any iterable, stages them in pinned memory and, on a
GPU, starts the host-to-device copy on a side stream so that it overlaps the previous step's kernels.

Reference counterpart: the DataLoader worker/pin-memory settings of tools/train/core.py:1728-1790 (``num_workers``,
``pin_memory``, ``prefetch_factor``); the copy to the device there happens synchronously at the top of the step
(core.py:2890-2900).  An exception raised by the source (an unreadable shard, a bad record) is carried to the
consumer and re-raised at the ``next()`` that would have returned that batch, never swallowed by the thread."""
from __future__ import annotations

import queue
import threading
from typing import Any, Dict, Iterable, Iterator, Optional

import torch

_END = object()


class _Failure:
    def __init__(self, exc: BaseException):
        self.exc = exc


class PiscesLxPrefetchLoader:
    def __init__(self, source: Iterable[Dict[str, Any]], depth: int = 2, device: Optional[torch.device] = None,
                 pin: bool = True):
        self.source, self.depth = source, max(1, depth)
        self.device = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available()
                                 else torch.device("cpu"))
        self.cuda = self.device.type == "cuda"
        self.pin = pin and self.cuda
        self._stream = torch.cuda.Stream(self.device) if self.cuda else None

    def _stage(self, batch: Dict[str, Any]) -> Dict[str, Any]:
        out: Dict[str, Any] = {}
        for k, v in batch.items():
            if not torch.is_tensor(v):
                out[k] = v
                continue
            if self.pin and not v.is_pinned() and v.device.type == "cpu":
                v = v.pin_memory()
            if self.cuda:
                with torch.cuda.stream(self._stream):
                    v = v.to(self.device, non_blocking=True)
            out[k] = v
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record(self._stream)
            out["__ready__"] = ev
        return out

    def __iter__(self) -> Iterator[Dict[str, Any]]:
        q: "queue.Queue[Any]" = queue.Queue(self.depth)
        stop = threading.Event()

        def put(item: Any) -> bool:
            while not stop.is_set():
                try:
                    q.put(item, timeout=0.1)
                    return True
                except queue.Full:
                    continue
            return False

        def work() -> None:
            try:
                if self.cuda:
                    torch.cuda.set_device(self.device)
                for b in self.source:
                    if not put(self._stage(b)):
                        return
                put(_END)
            except BaseException as e:                    # delivered to the consumer in order
                put(_Failure(e))

        t = threading.Thread(target=work, daemon=True, name="yv-prefetch")
        t.start()
        try:
            while True:
                item = q.get()
                if item is _END:
                    return
                if isinstance(item, _Failure):
                    raise item.exc
                ev = item.pop("__ready__", None)
                if ev is not None:
                    torch.cuda.current_stream(self.device).wait_event(ev)
                yield item
        finally:
            stop.set()
