"""An MPI communicator as the control plane (the reference's MPI bootstrap, ``deep_ep/_runtime.py:94-104`` there): the
library only needs ``Get_rank`` / ``Get_size`` / ``allgather`` / ``Barrier``, so a stand-in communicator that joins two
threads of this process serves as the test double.  Two ranks dispatch and combine through it on the CPU engine."""
import threading

import pytest
import torch

import deepep_b200 as deep_ep
from deepep_b200.oracle import reference as R
from deepep_b200.parallel.runtime import ControlPlane
from helpers import bits_equal, make_routes, make_weights


class World:
    def __init__(self, size):
        self.size, self.barrier, self.slots, self.lock = size, threading.Barrier(size), [None] * size, threading.Lock()


class Comm:
    """What mpi4py's ``MPI.Comm`` offers, for threads of one process."""

    def __init__(self, world, rank):
        self.world, self.rank = world, rank

    def Get_rank(self):
        return self.rank

    def Get_size(self):
        return self.world.size

    def Barrier(self):
        self.world.barrier.wait(timeout=30)

    def allgather(self, obj):
        self.world.slots[self.rank] = obj
        self.world.barrier.wait(timeout=30)
        out = list(self.world.slots)
        self.world.barrier.wait(timeout=30)
        return out


def test_control_plane_over_a_communicator():
    world = World(1)
    control = ControlPlane(Comm(world, 0))
    assert (control.rank, control.size, control.backend()) == (0, 1, "mpi") and control.all_gather_object("a") == ["a"]
    control.barrier()
    with pytest.raises(ValueError, match="contradicts"):
        ControlPlane(Comm(world, 0), rank=1)


def test_two_ranks_through_a_communicator():
    if torch.cuda.is_available():
        pytest.skip("CPU-engine test")
    T, H, E, K = [20, 7], 64, 4, 2
    xs = [torch.randn((T[r], H), generator=torch.Generator().manual_seed(r)).bfloat16() for r in range(2)]
    idx = [make_routes("invalid", T[r], E, K, 2, 9 + r) for r in range(2)]
    ws = [make_weights(T[r], K, r) for r in range(2)]
    ref, lays = R.dispatch(xs, idx, ws, E, do_expand=True)
    cref = R.combine([r[0] for r in ref], lays, T, K)
    world, results = World(2), {}

    def rank_main(rank):
        try:
            buf = deep_ep.ElasticBuffer(Comm(world, rank), num_max_tokens_per_rank=32, hidden=H, num_topk=K, explicitly_destroy=True,
                                        device="cpu", debug_collectives=True)
            rx, _, rw, handle, _ = buf.dispatch(xs[rank], topk_idx=idx[rank], topk_weights=ws[rank], num_experts=E, do_expand=True)
            out, _, _ = buf.combine(rx, handle)
            results[rank] = (buf.control.backend() == "mpi" and bits_equal(rx, ref[rank][0]) and bits_equal(rw, ref[rank][2])
                             and bits_equal(out, cref[rank][0]))
            buf.destroy()
        except Exception as exc:      # surfaced by the parent thread
            results[rank] = repr(exc)
            world.barrier.abort()

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(2)]
    [t.start() for t in threads]
    [t.join(60) for t in threads]
    assert results == {0: True, 1: True}
