"""Parity of the CUDA path (through the C ABI) against the CPU oracle on the same seeded inputs.

Tolerances are the contract's: float32 results within 1e-4 relative, bf16-store variants within 2e-2
(normwise: max |diff| / max |reference| per tensor).  Index work (plans, orderings) is bit-exact and
checked on CPU in test_host_cpu.py.
"""
import os

import numpy as np
import pytest

import agpt_b200 as A
from oracle import pyoracle as O
from tests.helpers import TOL_BF16, TOL_F32, chain_tree, random_qkv, random_tree, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=[(1, True), (1, False), (0, True)], ids=["tensor", "tensor-chunked", "fma"])
def attn_impl(request):
    """Every test in this file runs against both kernel families of the native attention entry points, the tensor-core
    family with either of its two kernel pairs (whole tile resident / chunked)."""
    impl, whole_tile = request.param
    A.set_attn_impl(impl)
    A.set_attn_variant(whole_tile, 4)
    yield impl
    A.set_attn_impl(1)
    A.set_attn_variant(True, 4)


def _dev(x, cuda):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).to(cuda)


def _run_native(parent, H, hd, q, k, v, go, cuda, tile_m=64, bf16=False):
    """Forward + backward through the walker plan; inputs and outputs in the caller's node order."""
    import torch
    plan = A.WalkerPlan(parent, tile_m, 0)
    order = plan.dfs_to_node.astype(np.int64)
    dq_, dk_, dv_, dg_ = [_dev(x[order], cuda) for x in (q, k, v, go)]
    ks, vs = (A.kv_store_write_bf16(dk_), A.kv_store_write_bf16(dv_)) if bf16 else (dk_, dv_)
    out, lse = A.attn_forward(plan, dq_, ks, vs, H)
    gq, gk, gv = A.attn_backward(plan, dq_, ks, vs, out, lse, dg_, H)
    torch.cuda.synchronize()
    inv = plan.node_to_dfs.astype(np.int64)
    res = [t.cpu().numpy()[inv] for t in (out, lse, gq, gk, gv)]
    return plan, res


def _oracle(parent, H, hd, q, k, v, go):
    out, w, w_off, depth = O.attn_fwd(parent, H, hd, q, k, v, grouped=True)
    dq, dk, dv = O.attn_bwd(parent, H, hd, q, k, v, w, w_off, go)
    return out, dq, dk, dv, w, w_off, depth


def _bf16_round(x):
    import torch
    return torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()


CASES = [
    # n, max_depth, H, hd, tile, seed
    (1, 1, 1, 16, 64, 0),
    (63, 6, 2, 16, 64, 1),
    (64, 9, 4, 16, 32, 2),
    (65, 5, 2, 32, 64, 3),
    (700, 12, 4, 32, 64, 4),
    (1500, 40, 2, 64, 64, 5),
    (900, 20, 2, 64, 128, 6),
    (2500, 64, 8, 64, 64, 7),
    (3000, 33, 4, 32, 128, 8),
    (1200, 16, 4, 16, 128, 9),
]


@pytest.mark.parametrize("n,md,H,hd,tile,seed", CASES)
def test_attention_fwd_bwd_matches_oracle(cuda, n, md, H, hd, tile, seed):
    parent = random_tree(n, md, seed, roots=min(3, n))
    q, k, v, go = random_qkv(n, H * hd, seed + 100)
    ref_out, ref_dq, ref_dk, ref_dv, w, w_off, depth = _oracle(parent, H, hd, q, k, v, go)
    _, (out, lse, dq, dk, dv) = _run_native(parent, H, hd, q, k, v, go, cuda, tile)
    assert rel_err(out, ref_out) < TOL_F32
    assert rel_err(dq, ref_dq) < TOL_F32
    assert rel_err(dk, ref_dk) < TOL_F32
    assert rel_err(dv, ref_dv) < TOL_F32
    # lse against the oracle's weights: w_self = exp(s_self - lse)
    scale = 1.0 / np.sqrt(hd)
    for i in range(0, n, max(1, n // 50)):
        for h in range(H):
            sl = slice(h * hd, (h + 1) * hd)
            s_self = float(q[i, sl].astype(np.float64) @ k[i, sl].astype(np.float64)) * scale
            w_self = w[w_off[i] + (h + 1) * depth[i] - 1]
            assert abs(np.exp(s_self - lse[i, h]) - w_self) < 1e-4 * max(1.0, w_self)


def test_deep_unary_chain_and_wide_star(cuda):
    """Edge shapes: one chain as deep as the plan allows per tile row, and a root with many leaves."""
    H, hd = 2, 32
    for parent in (chain_tree(200), np.concatenate([[-1], np.zeros(299, np.int32)]).astype(np.int32),
                   np.full(130, -1, np.int32)):
        n = parent.size
        q, k, v, go = random_qkv(n, H * hd, 77)
        ref = _oracle(parent, H, hd, q, k, v, go)
        _, (out, lse, dq, dk, dv) = _run_native(parent, H, hd, q, k, v, go, cuda, 64)
        # without ancestors every softmax has one term, so dq and the ds part of dk are exactly zero in the
        # oracle; those are compared absolutely (floor 1 = the O(1) scale of the inputs)
        floor = 1.0 if (parent < 0).all() else 1e-2
        for got, want in zip((out, dq, dk, dv), ref[:4]):
            assert rel_err(got, want, floor) < TOL_F32


def test_config1_trie_attention(cuda):
    """The reference-CPU-sized case: 20k-char corpus, depth-8 radix trie, 4 heads x 16."""
    corpus = A.synth_markov_corpus(20_000, 65, 2, 0)
    trie = A.RadixTrie.build(corpus, 8)
    parent, token, depth, _ = trie.char_tree()
    n, H, hd = parent.size, 4, 16
    q, k, v, go = random_qkv(n, H * hd, 5)
    ref = _oracle(parent, H, hd, q, k, v, go)
    plan, (out, lse, dq, dk, dv) = _run_native(parent, H, hd, q, k, v, go, cuda, 64)
    assert plan.max_depth == 8
    for got, want in zip((out, dq, dk, dv), ref[:4]):
        assert rel_err(got, want) < TOL_F32


def test_golden_vectors(cuda):
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "attention_small.npz"))
    H, hd = int(g["H"]), int(g["hd"])
    _, (out, lse, dq, dk, dv) = _run_native(g["parent"], H, hd, g["q"], g["k"], g["v"], g["dout"], cuda, 64)
    for name, got in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
        assert rel_err(got, g[name]) < TOL_F32, name


@pytest.mark.parametrize("hd,tile", [(16, 64), (32, 64), (64, 64), (64, 128)])
def test_bf16_store(cuda, hd, tile):
    H, n = 4, 1800
    parent = random_tree(n, 24, 31)
    q, k, v, go = random_qkv(n, H * hd, 32)
    _, (out, lse, dq, dk, dv) = _run_native(parent, H, hd, q, k, v, go, cuda, tile, bf16=True)
    # within the bf16 tolerance of the float32 oracle ...
    ref = _oracle(parent, H, hd, q, k, v, go)
    for got, want in zip((out, dq, dk, dv), ref[:4]):
        assert rel_err(got, want) < TOL_BF16
    # ... and, against the oracle fed the rounded store, within what single TF32 products leave (the bf16-store
    # kernels do not compensate TF32 rounding: 2^-11 per operand, below the store's own 2^-9); the FMA family is exact
    ref_r = _oracle(parent, H, hd, q, _bf16_round(k), _bf16_round(v), go)
    for got, want in zip((out, dq, dk, dv), ref_r[:4]):
        assert rel_err(got, want) < 2e-3


def test_backward_is_bitwise_repeatable(cuda):
    import torch
    H, hd, n = 4, 32, 5000
    parent = random_tree(n, 30, 41)
    q, k, v, go = random_qkv(n, H * hd, 42)
    plan = A.WalkerPlan(parent, 64, 0)
    order = plan.dfs_to_node.astype(np.int64)
    tq, tk, tv, tg = [_dev(x[order], cuda) for x in (q, k, v, go)]
    out, lse = A.attn_forward(plan, tq, tk, tv, H)
    a = [t.clone() for t in A.attn_backward(plan, tq, tk, tv, out, lse, tg, H)]
    b = A.attn_backward(plan, tq, tk, tv, out, lse, tg, H)
    torch.cuda.synchronize()
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_size_independent_properties_at_scale(cuda):
    """Microbenchmark-shaped tree (200k nodes, depth 64, 8 heads x 64): properties that need no oracle.
    out is a convex combination of V rows; with V = const the output is that constant; dV summed over all
    nodes equals dO summed over all nodes (every query's weights sum to one); dK summed over keys of
    ds*q telescopes to zero against dq*k: sum_i dq_i.q_i == sum_a dk_a.k_a."""
    import torch
    parent = A.synth_tree(200_000, 64, 65, 0.35, 65, 4000, 3)
    n, H, hd = parent.size, 8, 64
    plan = A.WalkerPlan(parent, 64, 0)
    g = torch.Generator(device=cuda).manual_seed(1)
    q, k, v, go = [torch.randn((n, H * hd), device=cuda, generator=g) for _ in range(4)]
    ones = torch.ones_like(v) * 0.5
    out, lse = A.attn_forward(plan, q, k, ones, H)
    assert torch.allclose(out, ones, atol=1e-5)
    out, lse = A.attn_forward(plan, q, k, v, H)
    dq, dk, dv = A.attn_backward(plan, q, k, v, out, lse, go, H)
    torch.cuda.synchronize()
    assert torch.isfinite(out).all() and torch.isfinite(dq).all() and torch.isfinite(dk).all()
    a, b = dv.double().sum(0), go.double().sum(0)
    assert float((a - b).abs().max() / b.abs().max()) < 1e-4
    lhs = float((dq.double() * q.double()).sum())
    rhs = float((dk.double() * k.double()).sum())
    assert abs(lhs - rhs) < 1e-4 * max(abs(lhs), abs(rhs), 1.0)
    # sampled nodes against the oracle on their own chains
    pos = np.linspace(0, n - 1, 40).astype(np.int64)
    qh, kh, vh, gh = [t.cpu().numpy() for t in (q, k, v, go)]
    oh = out.cpu().numpy()
    for i in pos:
        chain, c = [], int(i)
        while c >= 0:
            chain.append(c)
            c = int(plan.parent_dfs[c])
        chain.reverse()
        m = len(chain)
        sub_parent = np.arange(-1, m - 1, dtype=np.int32)
        ro, _, _, _ = O.attn_fwd(sub_parent, H, hd, qh[chain], kh[chain], vh[chain], save_weights=False)
        assert rel_err(oh[i], ro[-1]) < TOL_F32
    del gh


@pytest.mark.parametrize("n,H,hd", [(3000, 4, 32), (3001, 8, 64), (77, 4, 6)])     # the last takes the two-column kernel
def test_rope_and_row_gather(cuda, n, H, hd):
    import torch
    rng = np.random.default_rng(9)
    x = rng.standard_normal((n, H * hd)).astype(np.float32)
    y = rng.standard_normal((n, H * hd)).astype(np.float32)
    pos = rng.integers(0, 128, size=n).astype(np.int32)
    cos, sin = A.rope_table(128, hd)
    rot = lambda m, inv=False: O.rope_apply(m.reshape(n * H, hd), np.repeat(pos, H), cos, sin, inverse=inv).reshape(n, -1)  # noqa: E731
    want = rot(x)
    tx = _dev(x, cuda)
    A.rope_(tx, _dev(pos, cuda), _dev(cos, cuda), _dev(sin, cuda), H)
    assert rel_err(tx.cpu().numpy(), want) < 1e-6
    A.rope_(tx, _dev(pos, cuda), _dev(cos, cuda), _dev(sin, cuda), H, inverse=True)
    assert rel_err(tx.cpu().numpy(), x) < 1e-5
    # two matrices in one launch: the same values as one at a time, both directions
    for inv in (False, True):
        ta, tb, t1 = _dev(x, cuda), _dev(y, cuda), _dev(y, cuda)
        A.rope_pair_(ta, tb, _dev(pos, cuda), _dev(cos, cuda), _dev(sin, cuda), H, inverse=inv)
        A.rope_(t1, _dev(pos, cuda), _dev(cos, cuda), _dev(sin, cuda), H, inverse=inv)
        assert torch.equal(tb, t1)
        assert rel_err(ta.cpu().numpy(), rot(x, inv)) < 1e-6 and rel_err(tb.cpu().numpy(), rot(y, inv)) < 1e-6
    idx = rng.permutation(n).astype(np.int32)
    got = A.gather_rows(_dev(x, cuda), _dev(idx, cuda))
    assert torch.equal(got.cpu(), torch.from_numpy(x[idx]))


@pytest.mark.parametrize("lam,iw,ce_only,mass", [(0.0, 1.0, False, None), (0.5, 0.7, False, "linear"),
                                                 (1.0, 1.0, True, "log"), (0.0, 0.25, False, "sqrt")])
def test_loss_per_query(cuda, lam, iw, ce_only, mass):
    corpus = A.synth_markov_corpus(4000, 65, 2, 13)
    trie = A.RadixTrie.build(corpus, 8)
    ids = np.arange(1, trie.radix_count, dtype=np.int32)
    el = trie.edge_len[ids]
    qoff = np.concatenate([[0], np.cumsum(el)]).astype(np.int32)
    q2n = np.repeat(np.arange(ids.size, dtype=np.int32), el)
    toks = np.concatenate([trie.edge_tok[trie.edge_off[r]:trie.edge_off[r + 1]] for r in ids]).astype(np.int32)
    V, T = 65, int(qoff[-1])
    logits = (np.random.default_rng(1).standard_normal((T, V)) * 2).astype(np.float32)
    mw = A.mass_weights(trie.edge_mass[ids], el, mass) if mass else None
    coff = trie.cnt_off.astype(np.int32)
    want_l, want_g = O.loss_per_query(logits, q2n, qoff, ids, toks, coff, trie.cnt_tok, trie.cnt_val, mw, lam, iw, ce_only)
    got_l, got_g = A.loss_per_query(_dev(logits, cuda), _dev(q2n, cuda), _dev(qoff, cuda), _dev(ids, cuda), _dev(toks, cuda),
                                    _dev(coff, cuda), _dev(trie.cnt_tok, cuda), _dev(trie.cnt_val, cuda),
                                    _dev(mw, cuda) if mw is not None else None, lam, iw, ce_only)
    assert rel_err(got_l.cpu().numpy(), want_l) < TOL_F32
    assert rel_err(got_g.cpu().numpy(), want_g) < TOL_F32


def test_loss_golden_and_per_node(cuda):
    gl = np.load(os.path.join(os.path.dirname(__file__), "golden", "loss_small.npz"))
    got_l, got_g = A.loss_per_query(*[_dev(gl[k], cuda) for k in ("logits", "q2n", "qoff", "radix_ids", "token_ids", "cnt_off",
                                                                    "cnt_tok", "cnt_val", "mass_w")],
                                    float(gl["lam"]), float(gl["iw"]), False)
    assert rel_err(got_l.cpu().numpy(), gl["loss"]) < TOL_F32 and rel_err(got_g.cpu().numpy(), gl["grad"]) < TOL_F32
    rng = np.random.default_rng(2)
    N, V = 500, 96
    logits = rng.standard_normal((N, V)).astype(np.float32)
    off, tok, val = [0], [], []
    for _ in range(N):
        m = int(rng.integers(0, 6))
        tok += sorted(int(t) for t in rng.choice(V, size=m, replace=False))
        val += [int(x) for x in rng.integers(1, 20, size=m)]
        off.append(len(tok))
    ids = rng.permutation(N).astype(np.int32)
    want_l, want_g = O.loss_per_node(logits, ids, off, tok, val)
    got_l, got_g = A.loss_per_node(_dev(logits, cuda), _dev(ids, cuda), _dev(np.array(off, np.int32), cuda),
                                   _dev(np.array(tok, np.int32), cuda), _dev(np.array(val, np.int32), cuda))
    assert rel_err(got_l.cpu().numpy(), want_l) < TOL_F32 and rel_err(got_g.cpu().numpy(), want_g) < TOL_F32


def _pack(parent, depth, k, v):
    n = parent.size
    kv_off = np.concatenate([[0], np.cumsum(depth)[:-1]]).astype(np.int32)
    kp = np.zeros((int(depth.sum()), k.shape[1]), np.float32)
    vp = np.zeros_like(kp)
    for i in range(n):
        c, row = i, kv_off[i] + depth[i] - 1
        while c >= 0:
            kp[row], vp[row] = k[c], v[c]
            c, row = parent[c], row - 1
    return kv_off, kp, vp


@pytest.mark.parametrize("hd", [16, 32, 64])
def test_legacy_leveled_kernels(cuda, hd):
    """cuda_batched_varlen_attention{,_backward} + unpack on the packed-prefix layout."""
    import torch
    H, n = 4, 600
    parent = random_tree(n, 12, 51)
    depth = O.tree_depth_fast(parent)
    q, k, v, go = random_qkv(n, H * hd, 52)
    kv_off, kp, vp = _pack(parent, depth, k, v)
    max_len = int(depth.max())
    scale = float(1.0 / np.sqrt(hd))
    want_o, want_w = O.packed_attn_fwd(q, kp, vp, kv_off, depth, H, hd, max_len, scale)
    tq, tk, tv, tg = [_dev(x, cuda) for x in (q, kp, vp, go)]
    to, tl = _dev(kv_off, cuda), _dev(depth.astype(np.int32), cuda)
    got_o, got_w = A.legacy_attention(tq, tk, tv, to, tl, H, hd, max_len, scale)
    assert rel_err(got_o.cpu().numpy(), want_o) < TOL_F32
    assert rel_err(got_w.cpu().numpy(), want_w) < TOL_F32
    un = torch.empty((n, H * hd), device=cuda)
    A.lib().cuda_unpack_batched_attn_output(got_o.data_ptr(), un.data_ptr(), n, H, hd)
    A.lib().cuda_sync()
    assert torch.equal(un.reshape(-1), got_o)
    want = O.packed_attn_bwd(q, kp, vp, want_w, go, kv_off, depth, H, hd, max_len, scale)
    got = A.legacy_attention_backward(tq, tk, tv, got_w, tg, to, tl, H, hd, max_len, scale)
    for g_, w_ in zip(got, want):
        assert rel_err(g_.cpu().numpy().reshape(-1), w_) < TOL_F32


def test_legacy_L_queries_kernels(cuda):
    """Radix chunk form: query j of a node attends its ancestors plus own-edge rows 0..j."""
    corpus = A.synth_markov_corpus(3000, 20, 2, 17)
    trie = A.RadixTrie.build(corpus, 10)
    rx = O.Radix(O.Leveled(corpus, 10))
    H, hd = 2, 32
    D = H * hd
    ids = np.arange(1, trie.radix_count, dtype=np.int32)
    el = trie.edge_len[ids]
    anc = (rx.anc_off[1:] - rx.anc_off[:-1])[ids].astype(np.int32)
    T = int(el.sum())
    qoff = np.concatenate([[0], np.cumsum(el)]).astype(np.int32)
    q2n = np.repeat(np.arange(ids.size, dtype=np.int32), el)
    kvl = (anc + el).astype(np.int32)
    kvo = np.concatenate([[0], np.cumsum(kvl)]).astype(np.int32)
    rng = np.random.default_rng(3)
    # K/V per char position; queries are laid out node by node (chunk order), not in char order
    kc = rng.standard_normal((trie.total_edge_chars, D)).astype(np.float32)
    vc = rng.standard_normal((trie.total_edge_chars, D)).astype(np.float32)
    q = rng.standard_normal((T, D)).astype(np.float32)
    go = rng.standard_normal((T, D)).astype(np.float32)
    kp = np.zeros((int(kvo[-1]), D), np.float32)
    vp = np.zeros_like(kp)
    for i, r in enumerate(ids):
        a = rx.anc_ids[rx.anc_off[r]:rx.anc_off[r + 1]]
        own = trie.edge_start[r] + np.arange(el[i])
        rows = np.concatenate([a, own])
        kp[kvo[i]:kvo[i + 1]] = kc[rows]
        vp[kvo[i]:kvo[i + 1]] = vc[rows]
    max_len = int(kvl.max())
    scale = float(1.0 / np.sqrt(hd))
    want_o, want_w = O.packed_attn_fwd(q, kp, vp, kvo, kvl, H, hd, max_len, scale, q2n, qoff)
    dev = lambda x: _dev(x, cuda)  # noqa: E731
    got_o, got_w = A.legacy_attention(dev(q), dev(kp), dev(vp), dev(kvo), dev(kvl), H, hd, max_len, scale, dev(q2n), dev(qoff))
    assert rel_err(got_o.cpu().numpy(), want_o) < TOL_F32 and rel_err(got_w.cpu().numpy(), want_w) < TOL_F32
    want = O.packed_attn_bwd(q, kp, vp, want_w, go, kvo, kvl, H, hd, max_len, scale, q2n, qoff)
    got = A.legacy_attention_backward(dev(q), dev(kp), dev(vp), got_w, dev(go), dev(kvo), dev(kvl), H, hd, max_len, scale,
                                      dev(q2n), dev(qoff))
    for g_, w_ in zip(got, want):
        assert rel_err(g_.cpu().numpy().reshape(-1), w_) < TOL_F32
    # the native tree form gives the same per-query outputs on the char tree
    parent, _, _, _ = trie.char_tree()
    char_of_q = np.concatenate([trie.edge_start[r] + np.arange(el[i]) for i, r in enumerate(ids)])
    qc = np.zeros_like(kc)
    qc[char_of_q] = q
    _, (out, _, _, _, _) = _run_native(parent, H, hd, qc, kc, vc, np.zeros_like(qc), cuda)
    assert rel_err(out[char_of_q], want_o.reshape(T, D)) < TOL_F32


def test_host_buffer_entry_point(cuda):
    H, hd, n = 4, 32, 2000
    parent = random_tree(n, 20, 61)
    q, k, v, go = random_qkv(n, H * hd, 62)
    plan = A.WalkerPlan(parent, 64, 0)
    order, inv = plan.dfs_to_node.astype(np.int64), plan.node_to_dfs.astype(np.int64)
    o, lse, dq, dk, dv = A.attn_fwd_bwd_host(plan, *[np.ascontiguousarray(x[order]) for x in (q, k, v, go)], H)
    ref = _oracle(parent, H, hd, q, k, v, go)
    for got, want in zip((o, dq, dk, dv), ref[:4]):
        assert rel_err(got[inv], want) < TOL_F32


def test_bad_arguments_are_reported_not_fatal(cuda):
    import torch
    plan = A.WalkerPlan(random_tree(100, 5, 1), 64, 0)
    x = torch.zeros((100, 24), device=cuda)
    with pytest.raises(A.AgptError, match="head_dim"):
        A.attn_forward(plan, x, x, x, 2)            # head_dim 12
    y = torch.zeros((100, 64), device=cuda)
    out, lse = A.attn_forward(plan, y, y, y, 2)
    with pytest.raises(A.AgptError, match="workspace"):
        A.attn_backward(plan, y, y, y, out, lse, y, 2, workspace=torch.empty(16, dtype=torch.uint8, device=cuda))
    # the context is still usable afterwards
    out2, _ = A.attn_forward(plan, y, y, y, 2)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("V", [7, 32, 64, 65, 96, 128, 200, 300, 1000])
def test_loss_vocab_sizes(cuda, V):
    """Every register/shared-memory variant of the loss kernel, endpoint and intermediate rows mixed."""
    rng = np.random.default_rng(V)
    n_nodes = 300
    el = rng.integers(1, 5, size=n_nodes).astype(np.int32)
    qoff = np.concatenate([[0], np.cumsum(el)]).astype(np.int32)
    T = int(qoff[-1])
    q2n = np.repeat(np.arange(n_nodes, dtype=np.int32), el)
    toks = rng.integers(0, V, size=T).astype(np.int32)
    off, tok, val = [0], [], []
    for _ in range(n_nodes + 1):                      # radix ids 1..n_nodes; id 0 has no counts
        m = int(rng.integers(0, min(V, 6) + 1)) if len(off) > 1 else 0
        tok += sorted(int(t) for t in rng.choice(V, size=m, replace=False))
        val += [int(x) for x in rng.integers(1, 50, size=m)]
        off.append(len(tok))
    ids = np.arange(1, n_nodes + 1, dtype=np.int32)
    logits = (rng.standard_normal((T, V)) * 3).astype(np.float32)
    mw = rng.uniform(0.2, 3.0, size=T).astype(np.float32)
    off, tok, val = np.array(off, np.int32), np.array(tok + [0], np.int32), np.array(val + [0], np.int32)
    want_l, want_g = O.loss_per_query(logits, q2n, qoff, ids, toks, off, tok, val, mw, 0.7, 0.5, False)
    got_l, got_g = A.loss_per_query(_dev(logits, cuda), _dev(q2n, cuda), _dev(qoff, cuda), _dev(ids, cuda), _dev(toks, cuda),
                                    _dev(off, cuda), _dev(tok, cuda), _dev(val, cuda), _dev(mw, cuda), 0.7, 0.5, False)
    assert rel_err(got_l.cpu().numpy(), want_l) < TOL_F32
    assert rel_err(got_g.cpu().numpy(), want_g) < TOL_F32


def test_chain_deeper_than_the_tensor_path_holds(cuda):
    """A 600-deep unary chain exceeds the key capacity of a tensor-core tile; the entry points fall back to the
    FMA kernels and stay correct."""
    H, hd = 2, 16
    parent = chain_tree(600)
    q, k, v, go = random_qkv(600, H * hd, 99)
    ref = _oracle(parent, H, hd, q, k, v, go)
    _, (out, lse, dq, dk, dv) = _run_native(parent, H, hd, q, k, v, go, cuda, 64)
    for got, want in zip((out, dq, dk, dv), ref[:4]):
        assert rel_err(got, want) < TOL_F32


def test_deep_pruned_trie_bf16_store(cuda):
    """Shape of the deep configuration in miniature: order-4 corpus, depth-128 trie, count<2 pruning from depth 4,
    bf16 KV store, 6 heads x 64."""
    corpus = A.synth_markov_corpus(800, 96, 4, 21)
    trie = A.RadixTrie.build(corpus, 128, prune_min_mass=2, prune_min_depth=4)
    rx = O.Radix(O.Leveled(corpus, 128), 1, 2, 4)
    assert trie.radix_count == rx.radix_count and np.array_equal(trie.edge_start, rx.edge_start)
    parent, token, depth, _ = trie.char_tree()
    assert depth.max() > 100
    n, H, hd = parent.size, 6, 64
    q, k, v, go = random_qkv(n, H * hd, 81)
    plan, (out, lse, dq, dk, dv) = _run_native(parent, H, hd, q, k, v, go, cuda, 64, bf16=True)
    ref = _oracle(parent, H, hd, q, k, v, go)
    for got, want in zip((out, dq, dk, dv), ref[:4]):
        assert rel_err(got, want) < TOL_BF16
    ref_r = _oracle(parent, H, hd, q, _bf16_round(k), _bf16_round(v), go)
    for got, want in zip((out, dq, dk, dv), ref_r[:4]):
        assert rel_err(got, want) < 2e-3         # single TF32 products on a bf16 store (see test_bf16_store)


def test_host_buffer_entry_point_multi_chunk(cuda):
    """Enough rows for several upload/compute/download chunks, with subtrees that span chunk boundaries (their
    dK/dV rows are downloaded again at the end) and nodes whose reduction needs the second pass."""
    H, hd = 4, 16
    parent = A.synth_tree(700_000, 20, 5, 0.3, 8, 100_000, 11)
    n = parent.size
    q, k, v, go = random_qkv(n, H * hd, 63)
    plan = A.WalkerPlan(parent, 64, 0)
    assert n * H * hd * 4 > 2 * (64 << 20) and plan.info.n_reduce_multi > 0
    order, inv = plan.dfs_to_node.astype(np.int64), plan.node_to_dfs.astype(np.int64)
    ins = [np.ascontiguousarray(x[order]) for x in (q, k, v, go)]
    o, lse, dq, dk, dv = A.attn_fwd_bwd_host(plan, *ins, H)
    ref = _oracle(parent, H, hd, q, k, v, go)
    for got, want in zip((o, dq, dk, dv), ref[:4]):
        assert rel_err(got[inv], want) < TOL_F32
    # second call on the same plan reuses the cached arena and gives the same bits
    o2, lse2, dq2, dk2, dv2 = A.attn_fwd_bwd_host(plan, *ins, H)
    assert np.array_equal(dk, dk2) and np.array_equal(dv, dv2) and np.array_equal(o, o2)


@pytest.mark.parametrize("rows,cols", [(1, 4), (1000, 64), (4097, 128), (513, 384), (77, 1024)])
def test_layer_norm_kernels(cuda, rows, cols):
    import torch
    rng = np.random.default_rng(cols)
    x = (rng.standard_normal((rows, cols)) * 2 + 0.5).astype(np.float32)
    gamma = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    beta = rng.standard_normal(cols).astype(np.float32)
    grad = rng.standard_normal((rows, cols)).astype(np.float32)
    wy, wn, ws = O.layer_norm_fwd(x, gamma, beta)
    wdx, wdg, wdb = O.layer_norm_bwd(grad, wn, ws, gamma)
    y, norm, sinv = A.layer_norm_forward(_dev(x, cuda), _dev(gamma, cuda), _dev(beta, cuda))
    assert rel_err(y.cpu().numpy(), wy) < TOL_F32 and rel_err(norm.cpu().numpy(), wn) < TOL_F32
    assert rel_err(sinv.cpu().numpy(), ws) < TOL_F32
    dg, db = torch.ones(cols, device=cuda), torch.full((cols,), 2.0, device=cuda)      # accumulated into
    dx = A.layer_norm_backward(_dev(grad, cuda), norm, sinv, _dev(gamma, cuda), dg, db)
    assert rel_err(dx.cpu().numpy(), wdx) < TOL_F32
    assert rel_err(dg.cpu().numpy() - 1.0, wdg) < TOL_F32 and rel_err(db.cpu().numpy() - 2.0, wdb) < TOL_F32
    # the gradient of the residual path added in the same pass (also in place: add is the output buffer of a first call)
    skip = rng.standard_normal((rows, cols)).astype(np.float32)
    dg3, db3 = torch.zeros(cols, device=cuda), torch.zeros(cols, device=cuda)
    dx3 = A.layer_norm_backward(_dev(grad, cuda), norm, sinv, _dev(gamma, cuda), dg3, db3, add=_dev(skip, cuda))
    assert rel_err(dx3.cpu().numpy(), wdx + skip) < TOL_F32 and rel_err(dg3.cpu().numpy(), wdg) < TOL_F32
    with pytest.raises(A.AgptError):
        A.layer_norm_backward(_dev(grad, cuda), norm, sinv, _dev(gamma, cuda), dg3, db3, add=_dev(skip[:, :cols // 2 or 1], cuda))
    # legacy symbols, in place, default stream
    g2, n2 = _dev(grad, cuda), norm.clone()
    dg2, db2 = torch.zeros(cols, device=cuda), torch.zeros(cols, device=cuda)
    A.lib().cuda_layer_norm_backward(g2.data_ptr(), n2.data_ptr(), sinv.data_ptr(), _dev(gamma, cuda).data_ptr(), g2.data_ptr(),
                                     dg2.data_ptr(), db2.data_ptr(), rows, cols)
    A.lib().cuda_sync()
    assert torch.equal(g2, dx) and rel_err(dg2.cpu().numpy(), wdg) < TOL_F32


@pytest.mark.parametrize("gemm_impl", [1, 0])
@pytest.mark.parametrize("shape", [(1000, 128, 128), (70001, 128, 512), (4099, 512, 128), (64, 32, 64), (3, 4, 8)])
def test_gemm_f32_tensor_core(shape, gemm_impl):
    """The three layouts of the float32-accurate tensor-core GEMM (projection, input gradient, weight gradient with
    K cut into slices) against float64 products; tolerance 1e-5 of the largest entry (float32 rounding of a
    length-K sum)."""
    import torch
    rows, din, dout = shape
    A.set_gemm_impl(gemm_impl)
    g = torch.Generator(device="cuda").manual_seed(rows)
    x = torch.randn(rows, din, device="cuda", generator=g)
    w = torch.randn(din, dout, device="cuda", generator=g)
    b = torch.randn(dout, device="cuda", generator=g)
    dy = torch.randn(rows, dout, device="cuda", generator=g)

    def close(got, want):
        assert float((got.double() - want).abs().max() / want.abs().max()) < 1e-5

    close(A.gemm_f32(x, w, bias=b), x.double() @ w.double() + b.double())
    close(A.gemm_f32(x, w), x.double() @ w.double())
    res = torch.randn(rows, dout, device="cuda", generator=g)
    close(A.gemm_f32(x, w, bias=b, relu=True), torch.relu(x.double() @ w.double() + b.double()))
    close(A.gemm_f32(x, w, bias=b, residual=res), x.double() @ w.double() + b.double() + res.double())
    close(A.gemm_f32(x, w, residual=res), x.double() @ w.double() + res.double())
    close(A.gemm_f32(dy, w, trans_b=True, bias=torch.ones(din, device="cuda"), relu=True),
          torch.relu(dy.double() @ w.double().t() + 1.0))
    close(A.gemm_f32(dy, w, trans_b=True), dy.double() @ w.double().t())
    # input gradients of several projections of the same rows: the running sum is the source matrix and the output
    acc = A.gemm_f32(dy, w, trans_b=True)
    w2 = torch.randn(din, dout, device="cuda", generator=g)
    same = A.gemm_f32(dy, w2, trans_b=True, residual=acc, out=acc)
    assert same.data_ptr() == acc.data_ptr()
    close(acc, dy.double() @ w.double().t() + dy.double() @ w2.double().t())
    want = x.double().t() @ dy.double()
    for split_k in (1, 2, 7, 64):
        got = A.gemm_f32(x, dy, trans_a=True, split_k=split_k)
        close(got, want)
        assert torch.equal(got, A.gemm_f32(x, dy, trans_a=True, split_k=split_k))      # repeatable bit for bit
    with pytest.raises(A.AgptError):
        A.gemm_f32(x, w.t().contiguous(), trans_a=True, trans_b=True)
    A.set_gemm_impl(1)


def test_device_status_word_is_clear(cuda):
    """Every bounded wait on the device completed: the status word stays 0 after the kernels above ran."""
    assert A.device_status() == 0


@pytest.mark.parametrize("n,vocab,order,depth", [(200, 3, 1, 12), (20_000, 65, 2, 8), (150_000, 65, 3, 32), (30_000, 300, 2, 10),
                                                   (40_000, 96, 4, 128)])
def test_trie_build_gpu_equals_host_builder(cuda, n, vocab, order, depth):
    """Suffix order on the GPU (bit-exact against a plain sort on the small case) and the trie assembled from it
    against the level-by-level host builder, array for array, with bigram keys and pruning."""
    from tests.helpers import assert_same_trie, suffix_order
    corpus = A.synth_markov_corpus(n, vocab, order, 17)
    if vocab == 300:
        corpus = np.random.default_rng(3).integers(0, 300, n).astype(np.int32)        # more symbols than one byte holds
    sa, lcp, ms = A.suffix_order_gpu(corpus, depth + 1)
    assert sorted(sa.tolist()) == list(range(n - 1)) and ms > 0
    if n <= 20_000:
        want_sa, want_lcp = suffix_order(corpus, depth + 1)
        assert np.array_equal(lcp, want_lcp)
        # equal keys may come in any order; compare the keys themselves
        key = lambda s: tuple(corpus[s:s + depth + 1].tolist())  # noqa: E731
        assert [key(s) for s in sa] == [key(s) for s in want_sa]
    for level, mass, mdepth in ((1, 1, 4), (2, 2, 4)):
        want = A.RadixTrie.build(corpus, depth, subtree_level=level, prune_min_mass=mass, prune_min_depth=mdepth)
        got = A.RadixTrie.build_gpu(corpus, depth, subtree_level=level, prune_min_mass=mass, prune_min_depth=mdepth)
        assert_same_trie(got, want)


@pytest.mark.parametrize("mode,acc", [("local_depth", 0), ("own_edge", 2), ("full", 1)])
@pytest.mark.parametrize("hd,tile", [(32, 64), (16, 64), (64, 128)])
def test_gradient_modes_match_oracle(cuda, mode, acc, hd, tile):
    """The reference's three dK/dV behaviours (persistent accumulators; accumulators dropped per depth,
    src/agpt/trie_walk_trainer.cr:189; own radix edge only, src/cuda/agpt_train.cu:5016-5020) on a radix trie whose
    edges span tile boundaries; dQ is the same in all of them."""
    import torch
    corpus = A.synth_markov_corpus(4000, 12, 2, 4)
    trie = A.RadixTrie.build(corpus, 24)
    parent, token, depth, radix_of = trie.char_tree()
    n, H = parent.size, 2
    q, k, v, go = random_qkv(n, H * hd, 91)
    out, w, w_off, _ = O.attn_fwd(parent, H, hd, q, k, v, grouped=True)
    ref_dq, ref_dk, ref_dv = O.attn_bwd(parent, H, hd, q, k, v, w, w_off, go, accumulate_ancestors=acc, edge_id=radix_of)
    full_dq = O.attn_bwd(parent, H, hd, q, k, v, w, w_off, go)[0]
    assert np.array_equal(ref_dq, full_dq)
    plan = A.WalkerPlan(parent, tile, 0)
    order, inv = plan.dfs_to_node.astype(np.int64), plan.node_to_dfs.astype(np.int64)
    tq, tk, tv, tg = [_dev(x[order], cuda) for x in (q, k, v, go)]
    ef = torch.from_numpy(A.edge_first_positions(radix_of[order])).to(cuda)
    o, lse = A.attn_forward(plan, tq, tk, tv, H)
    dq, dk, dv = A.attn_backward(plan, tq, tk, tv, o, lse, tg, H, grad_mode=mode, edge_first=ef)
    torch.cuda.synchronize()
    for got, want in zip((dq, dk, dv), (ref_dq, ref_dk, ref_dv)):
        assert rel_err(got.cpu().numpy()[inv], want) < TOL_F32
    if mode != "full":
        with pytest.raises(A.AgptError):
            A.attn_backward(plan, tq, tk, tv, o, lse, tg, H, grad_mode="own_edge")          # edge_first missing
        with pytest.raises(A.AgptError):
            A.attn_backward(plan, tq, tk, tv, o, lse, tg, H, grad_mode="ancestors")


def test_injected_repeats_deep_trie_bf16_store(cuda, attn_impl):
    """Miniature of the deep configuration: a corpus with injected verbatim repeats, depth-128 radix trie pruned at
    count < 2, bf16 KV store, 64-wide heads.  Chains reach depth 128, so a tile holds up to 191 keys (the chunked
    tensor-core kernels; the whole-tile kernels take neither a bf16 store nor 64-wide heads)."""
    corpus = A.synth_markov_corpus(6_000, 12, 2, 3, 6)
    trie = A.RadixTrie.build(corpus, 128, 1, 2, 1)
    parent, token, depth, _ = trie.char_tree()
    assert int(depth.max()) == 128 and parent.size > 50_000 and int((depth >= 100).sum()) > 5_000
    n, H, hd = parent.size, 2, 64
    q, k, v, go = random_qkv(n, H * hd, 41)
    plan, (out, lse, dq, dk, dv) = _run_native(parent, H, hd, q, k, v, go, cuda, 64, bf16=True)
    assert plan.max_depth == 128
    ref = _oracle(parent, H, hd, q, _bf16_round(k), _bf16_round(v), go)        # the oracle on the rounded store
    for got, want in zip((out, dq, dk, dv), ref[:4]):
        assert rel_err(got, want) < 2e-3
    ref32 = _oracle(parent, H, hd, q, k, v, go)                                # and within the bf16 tolerance of the float32 oracle
    for got, want in zip((out, dq, dk, dv), ref32[:4]):
        assert rel_err(got, want) < TOL_BF16
