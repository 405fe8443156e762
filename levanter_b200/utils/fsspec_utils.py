"""fsspec helpers (src/levanter/utils/fsspec_utils.py:24-78)."""
from __future__ import annotations

import asyncio
import os
import re

import fsspec
from fsspec.core import url_to_fs


def exists(url, **kwargs) -> bool:
    fs, path = url_to_fs(url, **kwargs)
    return fs.exists(path)


def mkdirs(path: str) -> None:
    fs, p = url_to_fs(path)
    fs.makedirs(p, exist_ok=True)


def remove(url: str, *, recursive: bool = False, **kwargs) -> None:
    fs, path = url_to_fs(url, **kwargs)
    fs.rm(path, recursive=recursive)


async def async_remove(url: str, *, recursive: bool = False, **kwargs) -> None:
    loop = asyncio.get_running_loop()
    await loop.run_in_executor(None, lambda: remove(url, recursive=recursive, **kwargs))


_BRACE = re.compile(r"\{([^{}]*)\}")


def _brace_expand(pattern: str) -> list[str]:
    m = _BRACE.search(pattern)
    if not m:
        return [pattern]
    body = m.group(1)
    options: list[str]
    rng = re.fullmatch(r"(-?\d+)\.\.(-?\d+)", body)
    if rng:
        a, b = rng.group(1), rng.group(2)
        width = max(len(a), len(b)) if (a.startswith("0") and len(a) > 1) or (b.startswith("0") and len(b) > 1) else 0
        lo, hi = int(a), int(b)
        step = 1 if hi >= lo else -1
        options = [str(i).zfill(width) for i in range(lo, hi + step, step)]
    else:
        options = body.split(",")
    out = []
    for o in options:
        out.extend(_brace_expand(pattern[: m.start()] + o + pattern[m.end():]))
    return out


def expand_glob(url: str):
    """Brace expansion, then filesystem glob; results keep the protocol prefix."""
    for candidate in _brace_expand(url):
        fs, path = url_to_fs(candidate)
        if any(ch in path for ch in "*?["):
            protocol = candidate.split("://")[0] + "://" if "://" in candidate else ""
            rooted = candidate[len(protocol):].startswith("/")
            for p in sorted(fs.glob(path)):
                p = str(p)
                if protocol and not p.startswith(protocol):
                    # (some filesystems list "/bucket/key" for "proto://bucket/key": give back the form that was asked for)
                    p = protocol + (p.lstrip("/") if not rooted else p)
                yield p
        else:
            yield candidate


def join_path(lhs: str, rhs: str) -> str:
    """Join paths; an ``rhs`` carrying a protocol is absolute, and mismatching protocols raise."""
    if "://" in rhs:
        lp = lhs.split("://")[0] if "://" in lhs else None
        rp = rhs.split("://")[0]
        if lp is not None and lp != rp and not rhs.startswith(lhs):
            raise ValueError(f"cannot join {lhs!r} and {rhs!r}: different protocols")
        return rhs
    return os.path.join(lhs, rhs)
