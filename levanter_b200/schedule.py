"""Step-indexed schedules and the batch-size schedule with cumulative data offsets
(src/levanter/schedule.py:24-145).  ``BatchSchedule`` is what makes data order a pure function of the step: the loader
asks which global example indices belong to step ``n`` and resumes without seeking."""
from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import Generic, List, Sequence, Set, TypeVar, Union

T = TypeVar("T")
BIG_INT = 2**63 - 1


@dataclass
class ScheduleStep(Generic[T]):
    start: int
    value: T


IntSchedule = List[ScheduleStep[int]]


def _is_schedule(x) -> bool:
    return isinstance(x, Sequence) and not isinstance(x, (str, bytes)) and len(x) > 0 and isinstance(x[0], ScheduleStep)


def value_at_step(schedule_or_t, step: int):
    """Value of a schedule (or a plain value) at ``step``: the entry with the largest ``start <= step``."""
    if not _is_schedule(schedule_or_t):
        return schedule_or_t
    best = None
    for s in schedule_or_t:
        if step >= s.start:
            best = s
    if best is None:
        raise ValueError(f"Step {step} isn't after any of the schedule steps.")
    return best.value


def validate_schedule_sorted(schedule: Sequence[ScheduleStep]):
    if len(schedule) == 0:
        raise ValueError("Schedule must have at least one step.")
    if schedule[0].start != 0:
        raise ValueError("Schedule must start at step 0.")
    for i in range(1, len(schedule)):
        if schedule[i].start < schedule[i - 1].start:
            raise ValueError(f"Schedule is not sorted at index {i}")


def distinct_values(schedule) -> Set:
    if not _is_schedule(schedule):
        return {schedule}
    return set(s.value for s in schedule)


@dataclass
class BatchSegment:
    start: int   # first step of the segment
    until: int   # first step after it (BIG_INT when open-ended)
    value: int   # batch size
    offset: int  # examples consumed before the segment starts


class BatchSchedule:
    def __init__(self, schedule: Union[int, IntSchedule]):
        self.schedule = schedule
        if isinstance(schedule, int):
            self.segments = [BatchSegment(0, BIG_INT, schedule, 0)]
        else:
            if len(schedule) == 0:
                raise ValueError("Batch schedule must have at least one step.")
            validate_schedule_sorted(schedule)
            self.segments = []
            total = 0
            for i, step in enumerate(schedule):
                until = BIG_INT if i == len(schedule) - 1 else schedule[i + 1].start
                self.segments.append(BatchSegment(step.start, until, step.value, total))
                if until < BIG_INT:
                    total += (until - step.start) * step.value

    def _segment(self, step: int) -> BatchSegment:
        for seg in self.segments:
            if seg.start <= step < seg.until:
                return seg
        return self.segments[-1]

    def batch_size_at_step(self, step: int) -> int:
        return self._segment(step).value

    def global_data_offset_by_step(self, step: int) -> int:
        seg = self._segment(step)
        return seg.offset + (step - seg.start) * seg.value

    def find_step_containing_offset(self, offset: int) -> int:
        for seg in self.segments:
            span = (seg.until - seg.start) * seg.value if seg.until < BIG_INT else BIG_INT
            if seg.offset <= offset < seg.offset + span:
                return seg.start + (offset - seg.offset) // seg.value
        raise ValueError(f"Offset {offset} is beyond the last defined segment.")

    def batch_indices_at_step(self, bn: int) -> range:
        seg = self._segment(bn)
        base = seg.offset + (bn - seg.start) * seg.value
        return range(base, base + seg.value)

    def unique_batch_sizes(self) -> Set[int]:
        return set(seg.value for seg in self.segments)
