"""
Host-side failure handling of the batch-parallel replicas (no GPU is involved, no GPU is ever faulted): one replica
raises between steps or dies without a word; the others finish their work and the launcher names the failed rank.
World size 2 and 3 on CPU processes.
"""

import os
import time

import pytest

from nunchaku_rocm_b200.replicas import ReplicaFailure, run_replicas


def _worker(rank, world, sync, fail_rank, mode):
    failed_at_start = sync.start()
    done = 0
    for step in range(4):
        if rank == fail_rank and step == 2:
            if mode == "raise":
                raise ValueError("injected failure between steps")
            os._exit(7)  # dies without reporting anything
        time.sleep(0.02)  # the replica's own work: no collective, nothing that waits on a peer
        done += 1
    failed_at_end = sync.finish()
    return {"steps": done, "failed_at_start": failed_at_start, "failed_at_end": failed_at_end}


@pytest.mark.parametrize("mode", ["raise", "die"])
def test_one_replica_fails_the_others_finish_and_the_launcher_names_it(mode):
    report = run_replicas(_worker, world=3, args=(1, mode), timeout=20.0)
    assert sorted(report.results) == [0, 2]
    assert all(r["steps"] == 4 and r["failed_at_start"] == [] for r in report.results.values())
    assert list(report.failed) == [1]
    assert ("injected failure" in report.failed[1]) if mode == "raise" else ("exit code 7" in report.failed[1])
    # the survivors learnt on the host who had failed, and did not hang on it
    assert all(r["failed_at_end"] == [1] for r in report.results.values())
    with pytest.raises(ReplicaFailure, match="rank 1"):
        report.raise_for_failures()


def test_all_replicas_succeed():
    report = run_replicas(_worker, world=2, args=(-1, "raise"), timeout=20.0)
    assert report.ok and sorted(report.results) == [0, 1]
    report.raise_for_failures()
