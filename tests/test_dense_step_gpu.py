"""The dense-step kernels either side of the trie attention (bias, ReLU, bias gradient, softmax, embedding, optimizer)
through the C ABI against the oracle's restatements; native forms and the reference's legacy symbols."""
import numpy as np
import pytest

import agpt_b200 as A
from oracle import pyoracle as O
from tests.helpers import rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-4            # float32 parity tolerance of the path, relative to the largest entry


@pytest.fixture(scope="module")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda", 0)


def _dev(a, cuda):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


@pytest.mark.parametrize("rows,cols", [(1, 4), (37, 65), (1000, 128), (70001, 512), (513, 384), (5, 1028)])
def test_bias_relu_and_column_sums(cuda, rows, cols):
    import torch
    rng = np.random.default_rng(rows * 31 + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    bias = rng.standard_normal(cols).astype(np.float32)
    grad = rng.standard_normal((rows, cols)).astype(np.float32)
    xd, bd, gd = _dev(x, cuda), _dev(bias, cuda), _dev(grad, cuda)
    want_y, _ = O.bias_relu(x, bias, False)
    want_h, want_mask = O.bias_relu(x, bias, True)
    assert np.array_equal(A.bias_act(xd, bd).cpu().numpy(), want_y)
    mask = torch.empty_like(xd)
    h = A.bias_act(xd, bd, relu=True, mask=mask)
    assert np.array_equal(h.cpu().numpy(), want_h) and np.array_equal(mask.cpu().numpy(), want_mask)
    want_g = O.relu_bwd(grad, want_mask)
    assert np.array_equal(A.relu_backward(gd, mask).cpu().numpy(), want_g)
    assert np.array_equal(A.relu_backward(gd, h).cpu().numpy(), want_g)         # the activation works as the mask
    # bias gradient, plain and accumulated with a scale
    sums, _ = A.col_sum(gd)
    assert rel_err(sums.cpu().numpy(), O.col_sum(grad)) < TOL
    acc = torch.full((cols,), 3.0, device=cuda)
    A.col_sum(gd, out=acc, scale=0.5, accumulate=True)
    assert rel_err(acc.cpu().numpy() - 3.0, 0.5 * O.col_sum(grad)) < TOL
    # ReLU backward fused with the bias gradient, in place; repeatable bit for bit
    g2 = gd.clone()
    s2, masked = A.col_sum(g2, act=h)
    assert masked is g2 and np.array_equal(g2.cpu().numpy(), want_g)
    assert rel_err(s2.cpu().numpy(), O.col_sum(want_g)) < TOL
    s3, _ = A.col_sum(gd.clone(), act=h)
    assert torch.equal(s2, s3)
    # legacy symbols, in place on the default stream
    L = A.lib()
    x2 = xd.clone()
    L.cuda_bias_add(x2.data_ptr(), bd.data_ptr(), rows, cols)
    x3, m3 = xd.clone(), torch.empty_like(xd)
    L.cuda_fused_bias_relu(x3.data_ptr(), bd.data_ptr(), x3.data_ptr(), m3.data_ptr(), rows, cols)
    g3 = gd.clone()
    L.cuda_relu_backward(g3.data_ptr(), m3.data_ptr(), g3.data_ptr(), rows * cols)
    L.cuda_sync()
    assert np.array_equal(x2.cpu().numpy(), want_y) and np.array_equal(x3.cpu().numpy(), want_h)
    assert np.array_equal(m3.cpu().numpy(), want_mask) and np.array_equal(g3.cpu().numpy(), want_g)


@pytest.mark.parametrize("rows,cols", [(1, 1), (33, 65), (4097, 96), (100, 700)])
def test_softmax_rows_and_backward(cuda, rows, cols):
    import torch
    rng = np.random.default_rng(cols)
    x = (rng.standard_normal((rows, cols)) * 3).astype(np.float32)
    ds = rng.standard_normal((rows, cols)).astype(np.float32)
    s = A.softmax_rows(_dev(x, cuda))
    assert rel_err(s.cpu().numpy(), O.softmax_rows(x)) < TOL
    r = A.softmax_backward(s, _dev(ds, cuda))
    assert rel_err(r.cpu().numpy(), O.softmax_bwd(s.cpu().numpy(), ds)) < TOL
    L = A.lib()
    s2, r2 = torch.empty_like(s), torch.empty_like(s)
    L.cuda_softmax_rows(_dev(x, cuda).data_ptr(), s2.data_ptr(), rows, cols)
    L.cuda_softmax_backward(s2.data_ptr(), _dev(ds, cuda).data_ptr(), r2.data_ptr(), rows, cols)
    L.cuda_sync()
    assert torch.equal(s, s2) and torch.equal(r, r2)


@pytest.mark.parametrize("n,d,vocab", [(1, 4, 3), (1000, 64, 65), (300001, 128, 65), (5000, 384, 96), (777, 130, 300)])
def test_embedding_gather_and_gradient(cuda, n, d, vocab):
    import torch
    rng = np.random.default_rng(n)
    emb = rng.standard_normal((vocab, d)).astype(np.float32)
    ids = rng.integers(0, vocab, n).astype(np.int32)
    ids[rng.integers(0, n, max(1, n // 50))] = 0                   # a hot symbol: many collisions
    grad = rng.standard_normal((n, d)).astype(np.float32)
    ed, idd, gd = _dev(emb, cuda), _dev(ids, cuda), _dev(grad, cuda)
    assert np.array_equal(A.embedding_gather(ed, idd).cpu().numpy(), emb[ids])
    want = O.embedding_grad(grad, ids, vocab)
    got = A.embedding_grad(gd, idd, vocab)
    assert rel_err(got.cpu().numpy(), want) < TOL
    assert torch.equal(got, A.embedding_grad(gd, idd, vocab))       # repeatable bit for bit
    acc = torch.ones((vocab, d), device=cuda)
    A.embedding_grad(gd, idd, vocab, out=acc, accumulate=True)
    assert rel_err(acc.cpu().numpy() - 1.0, want) < TOL
    L = A.lib()
    out2, acc2 = torch.empty((n, d), device=cuda), torch.zeros((vocab, d), device=cuda)
    L.cuda_embedding_gather(ed.data_ptr(), idd.data_ptr(), out2.data_ptr(), n, d)
    L.cuda_embedding_scatter_add(gd.data_ptr(), idd.data_ptr(), acc2.data_ptr(), n, d)
    L.cuda_sync()
    assert np.array_equal(out2.cpu().numpy(), emb[ids]) and rel_err(acc2.cpu().numpy(), want) < TOL


@pytest.mark.parametrize("kind", ["sgd", "momentum", "rmsprop", "adam"])
@pytest.mark.parametrize("n,clip,wd", [(1, 0.0, 0.0), (1000, 0.5, 0.0), (300007, 0.0, 0.01), (300007, 2.0, 0.1), (4096, 1e9, 0.0)])
def test_optimizer_step(cuda, kind, n, clip, wd):
    """Three consecutive steps (state carried) against the float32 restatement; 1e-6 relative."""
    import torch
    rng = np.random.default_rng(n)
    p = rng.standard_normal(n).astype(np.float32)
    m = np.zeros(n, np.float32) if kind in ("momentum", "adam") else None
    v = np.zeros(n, np.float32) if kind in ("rmsprop", "adam") else None
    pd = _dev(p, cuda)
    md = None if m is None else _dev(m, cuda)
    vd = None if v is None else _dev(v, cuda)
    for t in (1, 2, 3):
        g = (rng.standard_normal(n) * 0.1).astype(np.float32)
        gd = _dev(g, cuda)
        p, m, v, norm = O.optimizer_step(kind, p, g, m, v, 3e-3, 0.9, 0.999, 1e-8, t, wd, clip)
        got_norm = A.optimizer_step(kind, pd, gd, md, vd, lr=3e-3, beta1=0.9, beta2=0.999, eps=1e-8, t=t, weight_decay=wd,
                                    clip_norm=clip, zero_grads=(t == 3))
        assert rel_err(pd.cpu().numpy(), p) < 1e-6
        if m is not None:
            assert rel_err(md.cpu().numpy(), m, floor=1e-6) < 1e-5
        if v is not None:
            assert rel_err(vd.cpu().numpy(), v, floor=1e-9) < 1e-5
        if clip > 0:
            assert abs(float(got_norm.item()) - norm) < 1e-5 * max(norm, 1.0)
        assert bool((gd == 0).all()) == (t == 3)


def test_optimizer_legacy_symbols_match_native(cuda):
    """clip -> update -> decay with the reference's symbols equals the native step bit for bit."""
    import torch
    n = 100003
    rng = np.random.default_rng(5)
    p0 = _dev(rng.standard_normal(n).astype(np.float32), cuda)
    g0 = _dev(rng.standard_normal(n).astype(np.float32), cuda)
    L = A.lib()
    for kind in ("sgd", "momentum", "rmsprop", "adam"):
        pa, ga, pb, gb = p0.clone(), g0.clone(), p0.clone(), g0.clone()
        ma, va, mb, vb = (torch.zeros(n, device=cuda) for _ in range(4))
        A.optimizer_step(kind, pa, ga, ma, va, lr=1e-2, beta1=0.9, beta2=0.99, eps=1e-8, t=1, weight_decay=0.05, clip_norm=1.5)
        partials, norm = torch.empty((n + 255) // 256, device=cuda), torch.empty(1, device=cuda)
        L.cuda_grad_clip_by_norm(gb.data_ptr(), 1.5, n, partials.data_ptr(), norm.data_ptr())
        if kind == "sgd":
            L.cuda_sgd_bulk(pb.data_ptr(), gb.data_ptr(), 1e-2, n)
        elif kind == "momentum":
            L.cuda_momentum_bulk(pb.data_ptr(), gb.data_ptr(), mb.data_ptr(), 1e-2, 0.9, n)
        elif kind == "rmsprop":
            L.cuda_rmsprop_bulk(pb.data_ptr(), gb.data_ptr(), vb.data_ptr(), 1e-2, 0.99, 1e-8, n)
        else:
            L.cuda_adam_bulk(pb.data_ptr(), gb.data_ptr(), mb.data_ptr(), vb.data_ptr(), 1e-2, 0.9, 0.99, 1e-8, 1, n)
        L.cuda_weight_decay(pb.data_ptr(), 1e-2, 0.05, n)
        L.cuda_sync()
        assert torch.equal(pa, pb), kind
        assert abs(float(norm.item()) - float(g0.double().norm().item())) < 1e-2
