"""Data-parallel host logic on CPU: two ranks as processes over gloo.

Each rank runs the host layer (tape, ready-gradient hand-off, trainer) on the numpy
stand-in backend with its own batch; the DataParallel object is replaced by one that sums
gradients with torch.distributed (gloo) instead of the library's NCCL communicator.  The
result must equal a single process that takes both batches as one step with 2 micro-steps
(sum of gradients scaled by 1/2), and both ranks must end with identical parameters.
"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class GlooDP:
    def __init__(self, world, rank):
        self.world, self.rank = world, rank
        self.handed = []

    def allreduce(self, grad):
        t = torch.from_numpy(np.array(grad.data, dtype=np.float32))
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        grad._host = t.numpy()
        self.handed.append(grad.shape)

    def wait(self):
        pass


class GlooBucketDP(GlooDP):
    """Same exchange through the bucket interface: small buckets so that several are flushed
    during backward and one at its end."""
    bucket_bytes = 8 << 10

    def __init__(self, world, rank):
        super().__init__(world, rank)
        self.buckets = []

    def allreduce_bucket(self, grads):
        self.buckets.append(len(grads))
        for g in grads:
            self.allreduce(g)


def _worker(rank, world, port, out_dir, bucketed=False, ckpt=False, wire="f32"):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from alpha2_b200.data import uniform_batches
    from alpha2_b200.gpt import ModelConfig
    from alpha2_b200.trainer import TrainConfig, Trainer
    from tests.fake_backend import NumpyBackend, T
    mc = ModelConfig(vocabSize=64, blockSize=16, nLayer=2, nEmbd=32, nHead=4, tied=True, init="plain")
    tc = TrainConfig(iters=10, batchSize=2, gradClip=0.5, seed=3)
    dp = GlooBucketDP(world, rank) if bucketed else GlooDP(world, rank)
    dp.wire = wire
    tr = Trainer(NumpyBackend(), mc, tc, dp=dp, activationCheckpointing=ckpt)
    batches = uniform_batches(100 + rank, 3, 2, 16, 64)          # a different stream per rank
    res = [tr.train_step([(T(t, "i32"), T(g, "i32"))]) for t, g in batches]
    n_params = len(tr.entries)
    assert len(dp.handed) == 3 * n_params                        # every gradient handed over once per step
    if bucketed:
        assert sum(dp.buckets) == 3 * n_params and len(dp.buckets) > 3 and max(dp.buckets) > 1
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), gn=np.array([r["gradNorm"] for r in res]),
             **{n: v.data.data for n, v in tr.entries})
    dist.destroy_process_group()


@pytest.mark.parametrize("bucketed,ckpt,wire", [(False, False, "f32"), (True, False, "f32"), (True, True, "f32"),
                                                 (True, False, "bf16")])
def test_two_ranks_equal_one_process_with_two_microsteps(tmp_path, bucketed, ckpt, wire):
    """``ckpt``: every block runs under activation checkpointing, where the block parameters'
    gradients are produced on an inner tape during the recompute; they must still all be
    handed to the exchange (the worker asserts one hand-over per parameter per step).
    ``wire="bf16"``: gradients travel as side copies that are converted back before the norm (the
    numpy stand-in keeps them in fp32, so this checks the plumbing; the rounding is checked on
    the GPU)."""
    port = 29500 + (os.getpid() + (997 if bucketed else 0) + (331 if ckpt else 0) + (173 if wire == "bf16" else 0)) % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path), bucketed, ckpt, wire), nprocs=2, join=True)
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    for k in r0.files:
        assert np.array_equal(r0[k], r1[k]), k                   # replicas stay identical
    from alpha2_b200.data import uniform_batches
    from alpha2_b200.gpt import ModelConfig
    from alpha2_b200.trainer import TrainConfig, Trainer
    from tests.fake_backend import NumpyBackend, T
    mc = ModelConfig(vocabSize=64, blockSize=16, nLayer=2, nEmbd=32, nHead=4, tied=True, init="plain")
    tr = Trainer(NumpyBackend(), mc, TrainConfig(iters=10, batchSize=2, gradClip=0.5, seed=3))
    b0, b1 = uniform_batches(100, 3, 2, 16, 64), uniform_batches(101, 3, 2, 16, 64)
    gns = []
    for i in range(3):
        pair = [(T(b0[i][0], "i32"), T(b0[i][1], "i32")), (T(b1[i][0], "i32"), T(b1[i][1], "i32"))]
        gns.append(tr.train_step(pair)["gradNorm"])
    np.testing.assert_allclose(r0["gn"], gns, rtol=2e-5)
    for n, v in tr.entries:
        np.testing.assert_allclose(r0[n], v.data.data, rtol=0, atol=2e-6, err_msg=n)
