"""Multi-rank path on CPU (gloo, world size 2): bigram-subtree sharding with context rows, per-rank
backward, one all-reduce of the projected gradient.  The kernels' role is played by the oracle here; what
is under test is the host logic the GPU ranks share: shard_tree, unit balance, and that summing the ranks'
gradients reproduces the unsharded gradient."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import agpt_b200 as A
from oracle import pyoracle as O
from tests.helpers import random_qkv, random_tree

H, HD, N = 2, 16, 1500


def _inputs():
    parent = random_tree(N, 10, 123, roots=5)
    q, k, v, go = random_qkv(N, H * HD, 124)
    x = np.random.default_rng(125).standard_normal((N, 24)).astype(np.float32)   # stand-in for the LN1 output
    return parent, q, k, v, go, x


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    parent, q, k, v, go, x = _inputs()
    lp, ids, ctx = A.shard_tree(parent, rank, world, level=2)
    ql, kl, vl, gl = q[ids], k[ids], v[ids], go[ids].copy()
    gl[ctx] = 0.0                                   # a context row is not trained on this rank
    out, w, w_off, _ = O.attn_fwd(lp, H, HD, ql, kl, vl)
    dq, dk, dv = O.attn_bwd(lp, H, HD, ql, kl, vl, w, w_off, gl)
    dq[ctx] = 0.0
    grad = torch.from_numpy(np.concatenate([x[ids].T @ dq, x[ids].T @ dk, x[ids].T @ dv], axis=1).astype(np.float64))
    dist.all_reduce(grad)
    owned = torch.tensor([int((~ctx).sum())])
    dist.all_reduce(owned)
    if rank == 0:
        ret["grad"] = grad.numpy()
        ret["owned"] = int(owned.item())
        ret["out_ids"] = ids[~ctx]
        ret["out"] = out[~ctx]
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gradient_equals_unsharded():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    parent, q, k, v, go, x = _inputs()
    out, w, w_off, _ = O.attn_fwd(parent, H, HD, q, k, v)
    dq, dk, dv = O.attn_bwd(parent, H, HD, q, k, v, w, w_off, go)
    want = np.concatenate([x.T @ dq, x.T @ dk, x.T @ dv], axis=1).astype(np.float64)
    assert ret["owned"] == N
    got = ret["grad"]
    assert np.abs(got - want).max() / np.abs(want).max() < 1e-5
    assert np.abs(ret["out"] - out[ret["out_ids"]]).max() < 1e-6


# ---- the trainer's epoch loop with two ranks: flat gradient buffer, statistics in its tail, one all-reduce ------------
class _FakeGroup:
    def __init__(self, grad, loss, count):
        self.grad, self.loss, self.count = grad, loss, count


class _FakeModel:
    """Stands in for TrieWalkModel on CPU: group_step adds a known gradient to the flat buffer and returns the loss
    statistics in the layout train_epoch expects."""

    def __init__(self, n_flat):
        self.n_flat = n_flat
        self.flat_grad = torch.zeros(n_flat + 4, dtype=torch.float32)
        self.device = torch.device("cpu")

    def bind_grads(self):
        pass

    def group_step(self, g, counts, sync=True, **kw):
        self.flat_grad[:self.n_flat] += g.grad
        n = torch.tensor(g.count)
        return torch.stack([torch.tensor(g.loss, dtype=torch.float32), (n // 4096).to(torch.float32), (n % 4096).to(torch.float32)])


class _FakeOpt:
    def __init__(self, model):
        self.model, self.seen = model, None

    def zero_grad(self, set_to_none=False):
        self.model.flat_grad.zero_()

    def step(self):
        self.seen = self.model.flat_grad[:self.model.n_flat].clone()
        self.model.flat_grad[:self.model.n_flat].zero_()


def _epoch_worker(rank, world, port, ret):
    from agpt_b200 import trainer as T
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    model = _FakeModel(10)
    opt = _FakeOpt(model)
    # counts far beyond 2^24 per rank: a float32 sum of them would not be exact
    groups = [_FakeGroup(torch.full((10,), float(rank + 1)), 2.5 * (rank + 1), 20_000_003 + rank),
              _FakeGroup(torch.arange(10, dtype=torch.float32), 1.25, 9_999_999)]
    loss, n_q = T.train_epoch(model, groups, None, opt, accumulate=True, world=world)
    if rank == 0:
        ret["loss"], ret["n_q"], ret["grad"] = loss, n_q, opt.seen.numpy()
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_epoch_sums_gradients_and_statistics_exactly():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_epoch_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret["n_q"] == (20_000_003 + 9_999_999) + (20_000_004 + 9_999_999)
    assert abs(ret["loss"] - (2.5 + 1.25 + 5.0 + 1.25)) < 1e-5
    assert np.array_equal(ret["grad"], (1.0 + 2.0) + 2 * np.arange(10, dtype=np.float32))
