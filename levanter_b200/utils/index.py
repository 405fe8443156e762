"""Bidirectional id <-> object map (src/levanter/utils/index.py:10-49)."""
from __future__ import annotations

from typing import Generic, Iterable, Iterator, Optional, TypeVar

T = TypeVar("T")


class Index(Generic[T]):
    def __init__(self, objs: Optional[Iterable[T]] = None):
        self._index_to_obj: list[T] = []
        self._obj_to_index: dict[T, int] = {}
        if objs is not None:
            for o in objs:
                self.append(o)

    def __len__(self) -> int:
        return len(self._index_to_obj)

    def get_index(self, obj: T) -> Optional[int]:
        return self._obj_to_index.get(obj)

    def get_obj(self, index: int) -> Optional[T]:
        return self._index_to_obj[index] if 0 <= index < len(self) else None

    def append(self, obj: T) -> int:
        idx = self._obj_to_index.get(obj)
        if idx is None:
            idx = len(self._index_to_obj)
            self._index_to_obj.append(obj)
            self._obj_to_index[obj] = idx
        return idx

    def __getitem__(self, index: int) -> T:
        return self._index_to_obj[index]

    def __contains__(self, obj: T) -> bool:
        return obj in self._obj_to_index

    def __iter__(self) -> Iterator[T]:
        return iter(self._index_to_obj)

    def index(self, obj: T) -> int:
        return self._obj_to_index[obj]
