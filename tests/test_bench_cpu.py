"""
Host-side logic of bench.py that does not need a GPU: the multi-rank aggregation (world size 2 over gloo), the reference
arm's rank rule, and the JSON contract of the reference arm on a tiny sample.
"""

import io
import json
import os
import sys
from contextlib import redirect_stdout

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench

    ms = bench.max_over_ranks(10.0 + 5.0 * rank, torch.device("cpu"))  # rank 1 is the slow one
    q.put((rank, ms, bench.whole_job_tops(world, 2.0e12, ms)))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_report_the_slowest_time_and_the_summed_throughput():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ms, tops in got:
        assert ms == 15.0                      # the maximum over ranks on every rank
        assert tops == pytest.approx(2 * 2.0e12 / 15e-3 / 1e12)  # two replicas' work in the slowest rank's time


def test_single_process_aggregation_is_the_identity():
    import bench

    assert bench.max_over_ranks(3.25, torch.device("cpu")) == 3.25
    assert bench.whole_job_tops(1, 1.0e12, 1000.0) == pytest.approx(1.0)


def test_reference_arm_runs_on_rank_zero_only(monkeypatch):
    import bench

    class Args:
        gpus, steps, warmup = 2, 1, 0

    monkeypatch.setenv("RANK", "1")
    buf = io.StringIO()
    with redirect_stdout(buf):
        bench.run_reference(Args())
    assert buf.getvalue() == ""


def test_reference_arm_line_has_the_contract_keys(monkeypatch):
    import bench

    class Args:
        gpus, steps, warmup = 1, 1, 0

    monkeypatch.setenv("RANK", "0")
    monkeypatch.setattr(bench, "cpu_baseline", lambda **kw: dict(value=0.1, unit="TOPS", cores=1, kind="port", sample="stub", ms_per_step=1.0))
    buf = io.StringIO()
    with redirect_stdout(buf):
        bench.run_reference(Args())
    line = json.loads(buf.getvalue())
    assert line["impl"] == "reference" and line["cpu_baseline"]["kind"] == "port"
    assert line["e2e"] == {"value": 0.1, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    for k in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "config"):
        assert k in line
