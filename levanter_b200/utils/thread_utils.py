"""Threads and asyncio glue (src/levanter/utils/thread_utils.py:14-101)."""
from __future__ import annotations

import asyncio
import threading
from concurrent.futures import ThreadPoolExecutor
from typing import AsyncIterator, Iterator, TypeVar

T = TypeVar("T")
_executor = ThreadPoolExecutor(max_workers=10)


def blocking_wait(coro):
    """Run a coroutine to completion from synchronous code, also when an event loop is already running."""
    try:
        loop = asyncio.get_running_loop()
    except RuntimeError:
        loop = None
    if loop is not None and loop.is_running():
        return _executor.submit(lambda: asyncio.run(coro)).result()
    return asyncio.run(coro)


class AsyncIteratorWrapper(Iterator[T]):
    """Synchronous iterator over an async iterator, driven by a private event-loop thread."""

    def __init__(self, async_iter: AsyncIterator[T]):
        self.async_iter = async_iter
        self.loop = asyncio.new_event_loop()
        self.thread = threading.Thread(target=self._run_loop, daemon=True)
        self.thread.start()
        self._exhausted = False

    def _run_loop(self):
        asyncio.set_event_loop(self.loop)
        self.loop.run_forever()

    def __iter__(self):
        return self

    def __next__(self):
        if self._exhausted:
            raise StopIteration
        fut = asyncio.run_coroutine_threadsafe(self.async_iter.__anext__(), self.loop)
        try:
            return fut.result()
        except StopAsyncIteration:
            self._exhausted = True
            self.close()
            raise StopIteration

    def close(self):
        if self.loop.is_running():
            self.loop.call_soon_threadsafe(self.loop.stop)


class ExceptionTrackingThread(threading.Thread):
    """Thread whose exception is re-raised by ``join``."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._exception = None

    def run(self):
        try:
            super().run()
        except BaseException as e:  # noqa: BLE001
            self._exception = e

    def join(self, timeout=None):
        super().join(timeout)
        if self._exception is not None:
            raise self._exception

    def check_raise(self):
        if self._exception is not None:
            raise self._exception
