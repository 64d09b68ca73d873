"""The allocation-free backward entry point (agpt_b200_attn_bwd_static).

It exists for callers that cannot get device memory when the backward pass runs -- a runtime that owns
the whole GPU and sub-allocates from its own pool, or a step with a frozen buffer set -- so its scratch is
an array built into the library.  The test calls it through the C ABI twice in a row (the array keeps the
first call's contents, which must not leak into the second) and compares every output with the workspace
variant, at the float32 parity tolerance; it also checks that a plan too large for the array is refused.
This file sorts last so that a run stopping at the first failure has already run everything else.
"""
import numpy as np
import pytest

import agpt_b200 as A
from tests.helpers import TOL_F32, random_qkv, random_tree, rel_err

pytestmark = pytest.mark.gpu


def _dev(x, cuda):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).to(cuda)


def test_static_scratch_backward_matches_workspace_backward(cuda):
    import torch
    H, hd = 4, 32
    cases = [(random_tree(6000, 30, 71), 72), (random_tree(2500, 12, 73), 74)]   # two different trees, back to back
    for parent, seed in cases:
        n = parent.size
        plan = A.WalkerPlan(parent, 64, 0)
        assert plan.workspace_bytes(H * hd) <= A.static_scratch_bytes()
        order = plan.dfs_to_node.astype(np.int64)
        q, k, v, go = [_dev(x[order], cuda) for x in random_qkv(n, H * hd, seed)]
        out, lse = A.attn_forward(plan, q, k, v, H)
        want = [t.clone() for t in A.attn_backward(plan, q, k, v, out, lse, go, H)]
        got = [torch.full_like(q, float("nan")) for _ in range(3)]     # pre-allocated by the caller
        A.attn_backward_static(plan, q, k, v, out, lse, go, H, *got)
        torch.cuda.synchronize()
        for g, w in zip(got, want):
            assert rel_err(g.cpu().numpy(), w.cpu().numpy()) < TOL_F32
        # second call on the same plan: the array still holds the first call's rows
        again = [torch.full_like(q, float("nan")) for _ in range(3)]
        A.attn_backward_static(plan, q, k, v, out, lse, go, H, *again)
        torch.cuda.synchronize()
        for g, w in zip(again, want):
            assert rel_err(g.cpu().numpy(), w.cpu().numpy()) < TOL_F32


def test_static_scratch_rejects_oversized_plan(cuda):
    import torch
    H, hd = 8, 64
    parent = A.synth_tree(400_000, 64, 65, 0.35, 65, 8000, 5)
    plan = A.WalkerPlan(parent, 64, 0)
    assert plan.workspace_bytes(H * hd) > A.static_scratch_bytes()
    x = torch.zeros((4, H * hd), device=cuda)       # never touched: the size check comes first
    with pytest.raises(A.AgptError, match="scratch"):
        A.attn_backward_static(plan, x, x, x, x, x, x, H, x, x, x)
