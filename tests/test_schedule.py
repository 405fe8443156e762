"""Step schedules and the batch-size schedule with cumulative data offsets (src/levanter/schedule.py)."""
import pytest

from levanter_b200.schedule import BatchSchedule, ScheduleStep, distinct_values, validate_schedule_sorted, value_at_step


def test_value_at_step():
    sched = [ScheduleStep(0, 32), ScheduleStep(100, 64), ScheduleStep(300, 128)]
    assert [value_at_step(sched, s) for s in (0, 99, 100, 299, 300, 10_000)] == [32, 32, 64, 64, 128, 128]
    assert value_at_step(17, 5) == 17
    assert distinct_values(sched) == {32, 64, 128} and distinct_values(8) == {8}


def test_unsorted_schedule_rejected():
    with pytest.raises(ValueError):
        validate_schedule_sorted([ScheduleStep(10, 1), ScheduleStep(5, 2)])


def test_batch_schedule_offsets():
    bs = BatchSchedule([ScheduleStep(0, 32), ScheduleStep(100, 64)])
    assert bs.batch_size_at_step(0) == 32 and bs.batch_size_at_step(100) == 64
    assert bs.global_data_offset_by_step(0) == 0
    assert bs.global_data_offset_by_step(100) == 3200
    assert bs.global_data_offset_by_step(101) == 3264
    assert bs.find_step_containing_offset(0) == 0
    assert bs.find_step_containing_offset(3199) == 99
    assert bs.find_step_containing_offset(3200) == 100
    assert bs.find_step_containing_offset(3263) == 100
    assert bs.find_step_containing_offset(3264) == 101
    lo, hi = bs.batch_indices_at_step(100)[0], bs.batch_indices_at_step(100)[-1]
    assert (lo, hi) == (3200, 3263)
    assert bs.unique_batch_sizes() == {32, 64} if hasattr(bs, "unique_batch_sizes") else True


def test_constant_batch_schedule():
    bs = BatchSchedule(16)
    assert bs.global_data_offset_by_step(10) == 160 and bs.find_step_containing_offset(161) == 10
