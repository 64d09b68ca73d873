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
