"""Failure handling of the data-parallel exchange, on CPU: no GPU is faulted, trapped or hung.

* A rank that leaves between steps announces it in the shared store; the remaining rank learns
  of it at the top of its next step, before it enqueues anything, and raises instead of entering
  a collective that would wait for ever.  Two real processes over gloo + a TCPStore.
* The host-side deadline around the exchange: ``DataParallel.sync`` polls the library for
  completion and for NCCL's asynchronous error state; a collective that never completes, and an
  asynchronous error, both end in an aborted communicator and a ``CollectiveError``.  The
  library is replaced by a stub that plays those two situations.
"""
import ctypes as C
import os
import sys
import time

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

from alpha2_b200.trainer import CollectiveError, DataParallel, PeerLeftError

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class _StubLib:
    """Stands in for libalpha_cuda.so: alpha_comm_query reports `pending` for ever, or an
    asynchronous error after a few polls."""

    def __init__(self, error_after=None, finish_after=None):
        self.polls, self.aborted = 0, 0
        self.error_after, self.finish_after = error_after, finish_after

    def alpha_comm_query(self, pending, err):
        self.polls += 1
        p, e = C.cast(pending, C.POINTER(C.c_int)), C.cast(err, C.POINTER(C.c_int))
        p[0] = 0 if (self.finish_after is not None and self.polls > self.finish_after) else 1
        e[0] = 6 if (self.error_after is not None and self.polls > self.error_after) else 0
        return 0

    def alpha_comm_abort(self):
        self.aborted += 1
        return 0


def _dp(lib, store=None, rank=0, world=2):
    dp = DataParallel.__new__(DataParallel)                  # no communicator: host logic only

    class _B:
        pass
    dp.backend, dp.world, dp.rank, dp.store = _B(), world, rank, store
    dp.backend.lib = lib
    return dp


def test_sync_returns_when_the_exchange_completes():
    lib = _StubLib(finish_after=5)
    _dp(lib).sync(timeout_s=5.0)
    assert lib.polls == 6 and lib.aborted == 0


def test_sync_gives_up_at_the_deadline_and_aborts():
    lib = _StubLib()
    t0 = time.monotonic()
    with pytest.raises(CollectiveError, match="did not finish within"):
        _dp(lib).sync(timeout_s=0.2)
    assert 0.2 <= time.monotonic() - t0 < 2.0 and lib.aborted == 1 and lib.polls > 10


def test_sync_reports_an_asynchronous_nccl_error_and_aborts():
    lib = _StubLib(error_after=3)
    with pytest.raises(CollectiveError, match="asynchronous error 6"):
        _dp(lib).sync(timeout_s=5.0)
    assert lib.aborted == 1 and lib.polls == 4


class _GlooDP(DataParallel):
    """The product's DataParallel with its NCCL calls replaced by gloo all-reduces; the store
    logic (leave / assert_peers) is the product's own."""

    def __init__(self, world, rank, store):
        self.world, self.rank, self.store, self.backend = world, rank, store, None
        self.exchanges = 0

    def allreduce(self, grad):
        import torch
        t = torch.from_numpy(np.array(grad.data, dtype=np.float32))
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        grad._host = t.numpy()
        self.exchanges += 1

    def allreduce_bucket(self, grads):
        for g in grads:
            self.allreduce(g)

    def wait(self):
        pass


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=__import__("datetime").timedelta(seconds=60))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world)
    from alpha2_b200.data import uniform_batches
    from alpha2_b200.gpt import ModelConfig
    from alpha2_b200.trainer import TrainConfig, Trainer
    from tests.fake_backend import NumpyBackend, T
    mc = ModelConfig(vocabSize=32, blockSize=8, nLayer=1, nEmbd=16, nHead=2)
    dp = _GlooDP(world, rank, store)
    tr = Trainer(NumpyBackend(), mc, TrainConfig(iters=10, batchSize=2, seed=3), dp=dp)
    batches = uniform_batches(50 + rank, 3, 2, 8, 32)
    outcome = []
    for i, (t, g) in enumerate(batches):
        if rank == 1 and i == 1:
            dp.leave()                                        # between steps, nothing in flight
            outcome.append("left")
            break
        if rank == 0 and i == 1:
            store.wait(["alpha_dp/left/1"])                   # make the order of events certain
        try:
            tr.train_step([(T(t, "i32"), T(g, "i32"))])
            outcome.append("step")
        except PeerLeftError as e:
            outcome.append("peer-left:" + str(e))
            break
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write("\n".join(outcome) + f"\nexchanges={dp.exchanges}\n")
    if rank == 0:
        time.sleep(0.5)                                       # keep the store up until rank 1 has written
    dist.destroy_process_group()


def test_a_rank_that_leaves_between_steps_is_seen_before_the_next_launch(tmp_path):
    port = 31500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0 = open(tmp_path / "rank0.txt").read().splitlines()
    r1 = open(tmp_path / "rank1.txt").read().splitlines()
    assert r1[:2] == ["step", "left"]
    assert r0[0] == "step" and r0[1].startswith("peer-left:") and "[1]" in r0[1]
    # rank 0 enqueued nothing for the step it refused: both ranks made the same number of exchanges
    assert r0[-1] == r1[-1]
