"""Host-side protocols of a tensor-parallel group on CPU ranks (gloo, world size 2 and 3): the collective decision on
the peer-memory exchange when one rank cannot map its peers, and what the others do when a rank leaves between
steps (they report instead of launching a step that would wait for it)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _agree_worker(rank, world, port, failing, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from rai_b200 import tp
    out[rank] = tp.agree_on_exchange(rank not in failing)
    dist.destroy_process_group()


@pytest.mark.parametrize("world,failing,want", [(2, (), True), (2, (1,), False), (3, (0,), False), (3, (), True)])
def test_every_rank_reaches_the_same_decision(world, failing, want):
    out = mp.Manager().dict()
    mp.spawn(_agree_worker, args=(world, _free_port(), failing, out), nprocs=world, join=True)
    assert [out[r] for r in range(world)] == [want] * world


def _leave_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from rai_b200 import tp
    store = dist.distributed_c10d._get_default_store()
    watch = tp.PeerWatch(store, rank, world, timeout_s=3.0)
    steps_done, reported = 0, None
    for step in range(6):
        if rank == world - 1 and step == 3:
            watch.leave()                 # between steps: nothing of this rank is in flight
            break
        try:
            watch.check(step)             # before the launch
        except tp.PeerLeft as e:
            reported = str(e)
            break
        t = torch.ones(1) * (rank + 1)    # the "step": a collective every member must join
        dist.all_reduce(t)
        steps_done += 1
    out[rank] = (steps_done, reported)
    # no barrier here: the leaving rank is gone; each rank tears down on its own
    dist.destroy_process_group()


def test_a_rank_that_leaves_between_steps_is_reported_not_waited_for():
    world = 2
    out = mp.Manager().dict()
    mp.spawn(_leave_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert out[1] == (3, None)                       # the leaving rank ran three steps and left quietly
    done, reported = out[0]
    assert done == 3 and reported and "left the group" in reported
