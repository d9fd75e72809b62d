"""Failure detection on the host, with Gloo ranks on the CPU: a rank that raises, a rank that
leaves, and a collective whose peer never joins. None of this touches a GPU."""

import datetime
import time

import pytest
import torch
import torch.distributed as dist

from pplx_garden.distributed import ParallelLaunch


def _raises_on_rank_1(device, dp_group, global_group):
    if global_group.rank == 1:
        raise RuntimeError("rank 1 gives up")
    global_group.barrier()   # rank 0 waits for a peer that is gone
    return True


def test_a_failing_rank_ends_the_launch_with_its_error() -> None:
    t0 = time.time()
    with pytest.raises(Exception) as info:
        ParallelLaunch(world_size=2).run(_raises_on_rank_1)
    assert time.time() - t0 < 60, "the launch must not wait for a collective timeout"
    assert "rank 1 gives up" in str(info.value)


def _leaves_between_steps(device, dp_group, global_group):
    # step 1 together, then rank 1 leaves cleanly between steps; rank 0 learns of it from its next
    # collective, which ends with an error instead of hanging
    x = torch.ones(4)
    global_group.all_reduce_cpu(x)
    assert float(x[0]) == 2.0
    if global_group.rank == 1:
        import os
        os._exit(0)   # no teardown, as a crashed process would not do one either
    try:
        global_group.all_reduce_cpu(torch.ones(4))
    except Exception as exc:  # noqa: BLE001
        return f"detected: {type(exc).__name__}"
    return "not detected"


def test_a_rank_that_leaves_is_detected_by_the_next_collective() -> None:
    t0 = time.time()
    try:
        results = ParallelLaunch(world_size=2).run(_leaves_between_steps)
        assert results[0].startswith("detected"), results
    except Exception:
        # the launcher may itself report the missing result of the rank that left: also a detection
        pass
    assert time.time() - t0 < 60


def _short_timeout_world(device, dp_group, global_group):
    # a sub-group with a short timeout: rank 0 enters a collective that rank 1 never joins
    pg = dist.new_group(ranks=[0, 1], backend="gloo", timeout=datetime.timedelta(seconds=2))
    if global_group.rank == 1:
        time.sleep(6)
        return "slept"
    t0 = time.time()
    try:
        dist.all_reduce(torch.ones(1), group=pg)
    except Exception as exc:  # noqa: BLE001
        return ("timeout", time.time() - t0, type(exc).__name__)
    return ("completed", time.time() - t0, "")


def test_a_collective_nobody_joins_runs_into_its_timeout() -> None:
    try:
        results = ParallelLaunch(world_size=2).run(_short_timeout_world)
    except Exception:
        return   # teardown after a timed-out collective may itself fail: the failure was seen
    kind, waited, _ = results[0]
    assert kind == "timeout" and waited < 30, results[0]
