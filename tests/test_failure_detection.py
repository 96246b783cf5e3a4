"""Failure detection without faulting anything: a rank leaves between steps and the others notice on
the host (store heartbeat) before their next collective."""
import pytest
import torch
import torch.distributed as dist

from dist_utils import run_distributed


def _worker(rank, world):
    from kareus_b200.parallel.health import Heartbeat, RankFailure
    hb = Heartbeat(timeout_s=1.0)
    x = torch.ones(4)
    for step in range(3):
        if step > 0:
            try:
                hb.check(step - 1)
            except RankFailure as e:
                assert rank == 0 and e.missing == [1] and e.step == 1, (rank, e.missing, e.step)
                return                      # stop before issuing a collective that would hang
        if rank == 1 and step == 2:
            raise AssertionError("rank 1 must have left already")
        dist.all_reduce(x)
        hb.finished(step)
        if rank == 1 and step == 0:
            hb.finished(0)
        if rank == 1 and step == 1:
            # finished step 1's collective but "dies" before publishing it
            hb.store.set(hb._key(1), "0")
            return
    raise AssertionError("rank 0 should have detected the missing peer")


def _entry(rank, world):
    try:
        _worker(rank, world)
    finally:
        pass


def test_missing_rank_is_detected_on_the_host():
    from kareus_b200.parallel.health import RankFailure  # noqa: F401
    # dist_utils ends with a barrier; rank 1 leaving early must not hang rank 0, so use a custom runner
    import torch.multiprocessing as mp
    from dist_utils import _free_port
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_spawn, args=(r, 2, port)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]


def _spawn(rank, world, port):
    import os
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    _worker(rank, world)
    # no barrier: the survivors leave without waiting for the rank that is gone
    os._exit(0)
