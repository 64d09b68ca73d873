"""The allocation-free backward entry point (agpt_b200_attn_bwd_static).

It exists for callers that cannot get device memory when the backward pass runs -- a runtime that owns
the whole GPU and sub-allocates from its own pool, or a step with a frozen buffer set -- so its scratch is
an array built into the library.  The test calls it through the C ABI twice in a row (the array keeps the
first call's contents, which must not leak into the second) and checks every output three ways: against the
CPU oracle at the parity tolerance, bit for bit against the workspace variant (both run the same kernels in
the same order), and that device memory in use does not change across a call.  It also checks that a plan
too large for the array is refused.  This file sorts last so that a run stopping at the first failure has
already run everything else.
"""
import numpy as np
import pytest

import agpt_b200 as A
from oracle import pyoracle as O
from tests.helpers import TOL_BF16, TOL_F32, random_qkv, random_tree, rel_err

pytestmark = pytest.mark.gpu


def _dev(x, cuda):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).to(cuda)


# (tree, seed, bf16 store, kernel family): the last tree has one root over 20000 rows, so its dK/dV row is
# reduced over more than 128 tiles and takes the two-pass (segment sum) path of the reduction
CASES = [
    ("two-pass reduction", lambda: random_tree(20000, 30, 75, roots=1), 76, False, 1),
    ("deep", lambda: random_tree(6000, 30, 71), 72, False, 1),
    ("shallow", lambda: random_tree(2500, 12, 73), 74, False, 1),
    ("bf16 store", lambda: random_tree(3000, 20, 77), 78, True, 1),
    ("fma kernels", lambda: random_tree(3000, 20, 79), 80, False, 0),
]


@pytest.mark.parametrize("name,make,seed,bf16,impl", CASES, ids=[c[0] for c in CASES])
def test_static_scratch_backward(cuda, name, make, seed, bf16, impl):
    import torch
    H, hd = 4, 32
    parent = make()
    n = parent.size
    A.set_attn_impl(impl)
    try:
        plan = A.WalkerPlan(parent, 64, 0)
        if name == "two-pass reduction":
            assert plan.info.n_reduce_multi > 0
        assert plan.workspace_bytes(H * hd) <= A.static_scratch_bytes()
        order, inv = plan.dfs_to_node.astype(np.int64), plan.node_to_dfs.astype(np.int64)
        hq, hk, hv, hg = random_qkv(n, H * hd, seed)
        q, k, v, go = [_dev(x[order], cuda) for x in (hq, hk, hv, hg)]
        if bf16:
            k, v = A.kv_store_write_bf16(k), A.kv_store_write_bf16(v)
        out, lse = A.attn_forward(plan, q, k, v, H)
        want = [t.clone() for t in A.attn_backward(plan, q, k, v, out, lse, go, H)]
        _, w, w_off, _ = O.attn_fwd(parent, H, hd, hq, hk, hv, grouped=True)
        ref = O.attn_bwd(parent, H, hd, hq, hk, hv, w, w_off, hg)
        got = [torch.full_like(q, float("nan")) for _ in range(3)]     # pre-allocated by the caller
        A.attn_backward_static(plan, q, k, v, out, lse, go, H, *got)   # first call on this device: address look-up
        torch.cuda.synchronize()
        # second call on the same plan: the array still holds the first call's rows; nothing may be allocated
        again = [torch.full_like(q, float("nan")) for _ in range(3)]
        torch.cuda.synchronize()
        free0, alloc0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        A.attn_backward_static(plan, q, k, v, out, lse, go, H, *again)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free0 and torch.cuda.memory_allocated() == alloc0
        tol = TOL_BF16 if bf16 else TOL_F32
        for res in (got, again):
            for g, w_, r in zip(res, want, ref):
                assert torch.equal(g, w_)                              # same kernels, same order: bit-equal
                assert rel_err(g.cpu().numpy()[inv], r) < tol
    finally:
        A.set_attn_impl(1)


def test_static_scratch_rejects_oversized_plan(cuda):
    import torch
    H, hd = 8, 64
    parent = A.synth_tree(400_000, 64, 65, 0.35, 65, 8000, 5)
    plan = A.WalkerPlan(parent, 64, 0)
    assert plan.workspace_bytes(H * hd) > A.static_scratch_bytes()
    x = torch.zeros((4, H * hd), device=cuda)       # never touched: the size check comes first
    with pytest.raises(A.AgptError, match="scratch"):
        A.attn_backward_static(plan, x, x, x, x, x, x, H, x, x, x)
    # the C entry point itself refuses too (the wrapper's check mirrors it)
    rc = A.lib().agpt_b200_attn_bwd_static(plan._h, x.data_ptr(), x.data_ptr(), x.data_ptr(), 0, x.data_ptr(), x.data_ptr(),
                                           x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), H, hd, 0.125, None)
    assert rc == -4 and b"scratch" in A.lib().agpt_b200_last_error()
