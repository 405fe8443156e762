"""Run a producer in a background thread and consume its items with bounded look-ahead.

Exceptions raised by the producer are re-raised in the consumer with the original traceback
(src/levanter/utils/background_iterable.py:92-166).
"""
from __future__ import annotations

import asyncio
import queue
import sys
import threading
from typing import AsyncIterator, Callable, Generic, Iterable, Iterator, Optional, TypeVar, Union

Ex = TypeVar("Ex")


class BackgroundIterable(Iterable[Ex]):
    def __init__(self, producer_fn: Callable[[], Union[Iterator[Ex], AsyncIterator[Ex]]], max_capacity: Optional[int] = None):
        self.max_capacity = max_capacity
        self._producer_fn = producer_fn

    def __iter__(self) -> "BackgroundIterator[Ex]":
        return BackgroundIterator(self._producer_fn, self.max_capacity)


class _End:
    pass


class _Err:
    def __init__(self, exc_info):
        self.exc_info = exc_info


class BackgroundIterator(Iterator[Ex]):
    def __init__(self, producer_fn, max_capacity: Optional[int]):
        self.max_capacity = max_capacity
        self._producer_fn = producer_fn
        self._stop_event = threading.Event()
        self.q: queue.Queue = queue.Queue(self.max_capacity or 0)
        self._done = False
        self.thread = threading.Thread(target=self._fill, daemon=True)
        self.thread.start()

    def __iter__(self):
        return self

    def __next__(self):
        if self._done:
            raise StopIteration
        while True:
            if self._stop_event.is_set() and self.q.empty():
                self._done = True
                raise StopIteration
            try:
                item = self.q.get(timeout=0.1)
            except queue.Empty:
                if not self.thread.is_alive() and self.q.empty():
                    self._done = True
                    raise StopIteration
                continue
            if isinstance(item, _End):
                self._done = True
                raise StopIteration
            if isinstance(item, _Err):
                self._done = True
                _, exc, tb = item.exc_info
                raise exc.with_traceback(tb)
            return item

    def __del__(self):
        self.stop()

    def stop(self, wait: bool = True):
        self._stop_event.set()
        if wait and threading.current_thread() is not self.thread:
            self.thread.join(timeout=1.0)

    def _put(self, item) -> bool:
        while not self._stop_event.is_set():
            try:
                self.q.put(item, timeout=0.1)
                return True
            except queue.Full:
                continue
        return False

    def _fill(self):
        try:
            it = self._producer_fn()
            if hasattr(it, "__anext__") or hasattr(it, "__aiter__"):
                asyncio.run(self._fill_async(it))
            else:
                for item in it:
                    if not self._put(item):
                        return
                self._put(_End())
        except BaseException:  # noqa: BLE001
            self._put(_Err(sys.exc_info()))

    async def _fill_async(self, it):
        ait = it.__aiter__() if hasattr(it, "__aiter__") else it
        async for item in ait:
            if not self._put(item):
                return
        self._put(_End())
