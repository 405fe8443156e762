"""Durations in config files (``"5m"``, ``"15min"``, ``"1d2h3m4.5s"``, ``"1:30:00"``).

Same grammar the reference accepts through pytimeparse (src/levanter/utils/datetime_utils.py:9-44).
"""
from __future__ import annotations

import re
from datetime import timedelta

_UNITS = {
    "w": 604800, "wk": 604800, "wks": 604800, "week": 604800, "weeks": 604800,
    "d": 86400, "day": 86400, "days": 86400,
    "h": 3600, "hr": 3600, "hrs": 3600, "hour": 3600, "hours": 3600,
    "m": 60, "min": 60, "mins": 60, "minute": 60, "minutes": 60,
    "s": 1, "sec": 1, "secs": 1, "second": 1, "seconds": 1,
    "ms": 1e-3, "msec": 1e-3, "millisecond": 1e-3, "milliseconds": 1e-3,
}
_TOKEN = re.compile(r"\s*([0-9]*\.?[0-9]+)\s*([a-zA-Z]+)?\s*,?")


def parse_seconds(s: str) -> float:
    s = s.strip()
    if not s:
        raise ValueError("empty duration")
    if re.fullmatch(r"[0-9]+(:[0-9]{1,2}){1,2}(\.[0-9]+)?", s):
        parts = [float(p) for p in s.split(":")]
        if len(parts) == 2:
            mnt, sec = parts
            return mnt * 60 + sec
        h, mnt, sec = parts
        return h * 3600 + mnt * 60 + sec
    total = 0.0
    pos = 0
    matched = False
    while pos < len(s):
        m = _TOKEN.match(s, pos)
        if not m or m.end() == pos:
            raise ValueError(f"cannot parse duration {s!r}")
        num = float(m.group(1))
        unit = (m.group(2) or "s").lower()
        if unit not in _UNITS:
            raise ValueError(f"unknown time unit {unit!r} in {s!r}")
        total += num * _UNITS[unit]
        pos = m.end()
        matched = True
    if not matched:
        raise ValueError(f"cannot parse duration {s!r}")
    return total


def parse_timedelta(td_str) -> timedelta:
    if isinstance(td_str, timedelta):
        return td_str
    if isinstance(td_str, (int, float)):
        return timedelta(seconds=float(td_str))
    td = timedelta(seconds=parse_seconds(str(td_str)))
    if td.total_seconds() < 0:
        raise ValueError("negative durations are not supported")
    return td


def encode_timedelta(td: timedelta) -> str:
    if td.total_seconds() < 0:
        raise ValueError("negative durations are not supported")
    out = ""
    if td.days:
        out += f"{td.days}d"
    seconds = td.seconds
    hours, seconds = divmod(seconds, 3600)
    minutes, seconds = divmod(seconds, 60)
    if hours:
        out += f"{hours}h"
    if minutes:
        out += f"{minutes}m"
    sec = seconds + td.microseconds / 1e6
    if sec or not out:
        out += f"{sec:g}s"
    return out
