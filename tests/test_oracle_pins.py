"""Pins of the CPU oracle: the reference's own known-answer constructions, restated.

* spec/agpt_backward_attention_spec.cr: the optimized backward routine and the explicit matrix
  formula agree to 1e-5 on a chain trie (prefix lengths 1..4) and on a branching depth batch, for
  dq, dk_cur, dv_cur, the ancestor accumulators and dWq/dWk/dWv; the attention output computed
  three ways agrees to 1e-5.
* rnd/sparsity-profile/README.md:97-101: radix endpoint / char-position counts of the real corpus.
* the committed golden vectors under tests/golden/.
"""
import os

import numpy as np
import pytest

from oracle import pyoracle as O
from tests.conftest import REFERENCE_ROOT
from tests.helpers import MemTrie, SpecModel, random_qkv, random_tree, rel_err

SPEC_TOL = 1e-5   # absolute, as in the reference spec
REF_CORPUS = os.path.join(REFERENCE_ROOT, "data", "input.txt")


def _spec_forward(model, trie, node_ids):
    """Post-RoPE q/k/v rows for the listed trie nodes (position = depth - 1), per-node ids kept."""
    H, hd = model.n_heads, model.hd
    cos, sin = O.rope_table(model.seq_len, hd)
    rows = {}
    for nid in node_ids:
        q, k, v, xn = model.qkv(trie.token[nid])
        pos = np.full(H, trie.depth[nid] - 1, np.int32)
        q = O.rope_apply(q.reshape(H, hd), pos, cos, sin).reshape(-1)
        k = O.rope_apply(k.reshape(H, hd), pos, cos, sin).reshape(-1)
        rows[nid] = (q, k, v, xn)
    return rows, cos, sin


def _check_node(model, rows, cos, sin, chain, d_attn_proj, prefix_len):
    """One node: formula A (matrix) vs formula B (optimized) exactly as the spec compares them."""
    H, hd, D = model.n_heads, model.hd, model.d_model
    nid = chain[-1]
    n = len(chain)
    # a private little tree: the chain itself
    parent = np.arange(-1, n - 1, dtype=np.int32)
    q = np.stack([rows[c][0] for c in chain])
    k = np.stack([rows[c][1] for c in chain])
    v = np.stack([rows[c][2] for c in chain])
    out, w, w_off, depth = O.attn_fwd(parent, H, hd, q, k, v)
    out_g, w_g, _, _ = O.attn_fwd(parent, H, hd, q, k, v, grouped=True)
    assert np.abs(out - out_g).max() <= SPEC_TOL and np.abs(w - w_g).max() <= SPEC_TOL
    d_concat = (d_attn_proj @ model.wo_w.T).astype(np.float32)
    pos = np.array([n - 1], np.int32)
    dq_all = {"old": np.zeros(D, np.float32), "new": np.zeros(D, np.float32)}
    dk_all = {"old": np.zeros(D, np.float32), "new": np.zeros(D, np.float32)}
    dv_all = {"old": np.zeros(D, np.float32), "new": np.zeros(D, np.float32)}
    for hi in range(H):
        sl = slice(hi * hd, (hi + 1) * hd)
        Kh, Vh = k[:, sl], v[:, sl]
        wh = w[w_off[n - 1] + hi * n: w_off[n - 1] + (hi + 1) * n]
        go = d_concat[sl]
        # attention output three ways: weights x V, explicit loop, saved forward output
        o_mat = (wh[None, :] @ Vh)[0]
        o_loop = np.zeros(hd, np.float32)
        for p in range(n):
            o_loop += wh[p] * Vh[p]
        assert np.abs(o_mat - o_loop).max() <= SPEC_TOL
        assert np.abs(o_mat - out[n - 1, sl]).max() <= SPEC_TOL
        assert abs(float(o_mat @ go) - float(o_loop @ go)) <= SPEC_TOL
        acc_dk = (0.001 * (prefix_len + hi + np.arange(hd) + 1)).astype(np.float32)
        acc_dv = (0.002 * (prefix_len + hi + np.arange(hd) + 1)).astype(np.float32)
        dq_o, dkf, dvf = O.bwd_head_matrix(Kh, Vh, wh, q[n - 1, sl], go, acc_dk, acc_dv)
        dq_n, dkc, dvc, anc_dk, anc_dv = O.bwd_head_optimized(Kh, Vh, wh, q[n - 1, sl], go, acc_dk, acc_dv,
                                                              np.zeros((max(n - 1, 1), hd), np.float32),
                                                              np.zeros((max(n - 1, 1), hd), np.float32))
        dq_o = O.rope_apply(dq_o[None, :], pos, cos, sin, inverse=True)[0]
        dq_n = O.rope_apply(dq_n[None, :], pos, cos, sin, inverse=True)[0]
        dk_o = O.rope_apply(dkf[n - 1][None, :], pos, cos, sin, inverse=True)[0]
        dk_n = O.rope_apply(dkc[None, :], pos, cos, sin, inverse=True)[0]
        assert np.abs(dq_o - dq_n).max() <= SPEC_TOL
        assert np.abs(dk_o - dk_n).max() <= SPEC_TOL
        assert np.abs(dvf[n - 1] - dvc).max() <= SPEC_TOL
        if n > 1:   # ancestor accumulators (they start at zero in both formulas)
            assert np.abs(dkf[:n - 1] - anc_dk[:n - 1]).max() <= SPEC_TOL
            assert np.abs(dvf[:n - 1] - anc_dv[:n - 1]).max() <= SPEC_TOL
        dq_all["old"][sl], dq_all["new"][sl] = dq_o, dq_n
        dk_all["old"][sl], dk_all["new"][sl] = dk_o, dk_n
        dv_all["old"][sl], dv_all["new"][sl] = dvf[n - 1], dvc
    xn = rows[nid][3]
    for g in (dq_all, dk_all, dv_all):
        assert np.abs(np.outer(xn, g["old"]) - np.outer(xn, g["new"])).max() <= SPEC_TOL
    return dq_all["new"], dk_all["new"], dv_all["new"]


def test_spec_chain_prefix_lengths():
    model = SpecModel()
    trie = MemTrie(list(range(8)), max_depth=6, max_starts=1)
    levels = trie.levels()
    assert [len(lv) for lv in levels[1:]] == [1] * 6 and [trie.token[lv[0]] for lv in levels[1:]] == list(range(6))
    rows, cos, sin = _spec_forward(model, trie, range(1, len(trie.parent)))
    for prefix_len in (1, 2, 3, 4):
        nid = levels[prefix_len][0]
        chain = []
        c = nid
        while c != 0:
            chain.append(c)
            c = trie.parent[c]
        chain.reverse()
        assert len(chain) == prefix_len
        d_attn_proj = (0.01 * (prefix_len + np.arange(model.d_model) + 1)).astype(np.float32)
        _check_node(model, rows, cos, sin, chain, d_attn_proj, prefix_len)


def test_spec_branching_depth_batch():
    model = SpecModel()
    toks = [0, 1, 2, 7, 0, 1, 3, 7, 0, 4, 2, 7, 0, 4, 3, 7]
    trie = MemTrie(toks, max_depth=4)
    levels = trie.levels()
    batch = levels[1]           # the first level with more than one node
    assert len(batch) > 1
    rows, cos, sin = _spec_forward(model, trie, range(1, len(trie.parent)))
    for i, nid in enumerate(batch):
        d_attn_proj = (0.005 * (i * model.d_model + np.arange(model.d_model) + 1)).astype(np.float32)
        _check_node(model, rows, cos, sin, [nid], d_attn_proj, 1)


def test_full_tree_backward_equals_per_node_formula():
    """The tree-level backward (deepest-first accumulation) equals summing the matrix formula's rows."""
    H, hd = 2, 16
    parent = random_tree(150, 7, seed=3)
    q, k, v, go = random_qkv(150, H * hd, seed=4)
    out, w, w_off, depth = O.attn_fwd(parent, H, hd, q, k, v)
    dq, dk, dv = O.attn_bwd(parent, H, hd, q, k, v, w, w_off, go)
    ref_dk = np.zeros_like(dk, dtype=np.float64)
    ref_dv = np.zeros_like(dv, dtype=np.float64)
    zeros = np.zeros(hd, np.float32)
    for i in range(150):
        chain = []
        c = i
        while c >= 0:
            chain.append(c)
            c = parent[c]
        chain.reverse()
        n = len(chain)
        for h in range(H):
            sl = slice(h * hd, (h + 1) * hd)
            wh = w[w_off[i] + h * n: w_off[i] + (h + 1) * n]
            dq_o, dkf, dvf = O.bwd_head_matrix(k[chain][:, sl], v[chain][:, sl], wh, q[i, sl], go[i, sl], zeros, zeros)
            assert np.abs(dq_o - dq[i, sl]).max() <= 1e-5
            for p, c in enumerate(chain):
                ref_dk[c, sl] += dkf[p]
                ref_dv[c, sl] += dvf[p]
    assert rel_err(dk, ref_dk) < 1e-5 and rel_err(dv, ref_dv) < 1e-5
    # units x heads in parallel give bit-identical results
    roots = np.nonzero(parent < 0)[0]
    dq2, dk2, dv2 = O.attn_bwd(parent, H, hd, q, k, v, w, w_off, go, unit_off=None)
    assert np.array_equal(dk, dk2) and np.array_equal(dq, dq2)
    # local-depth behaviour: ancestor rows dropped
    _, dk3, _ = O.attn_bwd(parent, H, hd, q, k, v, w, w_off, go, accumulate_ancestors=False)
    leaf = np.setdiff1d(np.arange(150), parent[parent >= 0])
    assert np.array_equal(dk3[leaf], dk[leaf])
    del roots


def test_grouped_matches_per_node():
    H, hd = 4, 16
    parent = random_tree(400, 9, seed=11)
    q, k, v, _ = random_qkv(400, H * hd, seed=12)
    o1, w1, off, _ = O.attn_fwd(parent, H, hd, q, k, v)
    o2, w2, _, _ = O.attn_fwd(parent, H, hd, q, k, v, grouped=True)
    assert rel_err(o2, o1) < 1e-6 and np.abs(w1 - w2).max() < 1e-6


def test_packed_layout_matches_tree():
    """The packed-prefix (legacy boundary) restatement equals the tree form on the same nodes."""
    H, hd = 2, 16
    parent = random_tree(120, 6, seed=21)
    n = parent.size
    q, k, v, go = random_qkv(n, H * hd, seed=22)
    out, w, w_off, depth = O.attn_fwd(parent, H, hd, q, k, v)
    kv_off = np.concatenate([[0], np.cumsum(depth)[:-1]]).astype(np.int32)
    kp = np.zeros((int(depth.sum()), H * hd), np.float32)
    vp = np.zeros_like(kp)
    for i in range(n):
        c, row = i, kv_off[i] + depth[i] - 1
        while c >= 0:
            kp[row], vp[row] = k[c], v[c]
            c, row = parent[c], row - 1
    max_len = int(depth.max())
    scale = np.float32(1.0 / np.sqrt(hd))
    po, pw = O.packed_attn_fwd(q, kp, vp, kv_off, depth, H, hd, max_len, scale)
    assert rel_err(po.reshape(n, -1), out) < 1e-6
    dq, dk, dv = O.attn_bwd(parent, H, hd, q, k, v, w, w_off, go)
    pdq, pdk, pdv = O.packed_attn_bwd(q, kp, vp, pw, go, kv_off, depth, H, hd, max_len, scale)
    assert rel_err(pdq.reshape(n, -1), dq) < 1e-6
    # scatter the packed rows back onto their tree nodes
    sk = np.zeros_like(dk, dtype=np.float64)
    pdk = pdk.reshape(-1, H * hd)
    for i in range(n):
        c, row = i, kv_off[i] + depth[i] - 1
        while c >= 0:
            sk[c] += pdk[row]
            c, row = parent[c], row - 1
    assert rel_err(sk, dk) < 1e-5


def test_loss_variants_agree():
    rng = np.random.default_rng(5)
    V, N = 65, 40
    logits = rng.standard_normal((N, V)).astype(np.float32) * 2
    cnt_off = [0]
    tok, val = [], []
    for i in range(N):
        m = int(rng.integers(0, 5))
        ts = rng.choice(V, size=m, replace=False)
        tok += sorted(int(t) for t in ts)
        val += [int(x) for x in rng.integers(1, 9, size=m)]
        cnt_off.append(len(tok))
    l_node, g_node = O.loss_per_node(logits, np.arange(N), cnt_off, tok, val)
    l_cr, g_cr = O.loss_crystal(logits, cnt_off, tok, val, 0.0)
    has = np.diff(cnt_off) > 0
    assert np.abs(l_node[has] - l_cr[has]).max() < 1e-5
    assert np.abs(g_node[has] - g_cr[has]).max() < 1e-6
    # every node an endpoint of a one-char edge: the per-query kernel reduces to the per-node one
    q2n = np.arange(N)
    qoff = np.arange(N + 1)
    l_q, g_q = O.loss_per_query(logits, q2n, qoff, np.arange(N), np.zeros(N, np.int32), cnt_off, tok, val)
    assert np.array_equal(l_q, l_node) and np.array_equal(g_q, g_node)
    # gradient rows of nodes with counts sum to zero (probabilities minus a distribution)
    assert np.abs(g_node[has].sum(axis=1)).max() < 1e-5


def _real_corpus_tokens():
    text = open(REF_CORPUS, "rb").read().decode("utf-8")
    vocab = {c: i for i, c in enumerate(sorted(set(text)))}
    return np.fromiter((vocab[c] for c in text), dtype=np.int32, count=len(text))


@pytest.mark.skipif(not os.path.exists(REF_CORPUS), reason="reference corpus not mounted")
@pytest.mark.parametrize("depth,endpoints,chars", [(8, 845_539, 1_545_081), (16, 1_607_927, 9_313_896)])
def test_real_corpus_trie_shape(depth, endpoints, chars):
    """Counts published for the reference's own corpus (rnd/sparsity-profile/README.md:97-101); the
    tokenizer is the sorted set of characters (src/agpt.cr:28)."""
    tok = _real_corpus_tokens()
    lv = O.Leveled(tok, depth)
    rx = O.Radix(lv)
    assert rx.radix_count - 1 == endpoints
    assert rx.total_edge_chars == chars
    if depth == 8:
        import agpt_b200 as A
        tr = A.RadixTrie.build(tok, depth)
        assert tr.radix_count - 1 == endpoints and tr.total_edge_chars == chars
        assert np.array_equal(tr.edge_start, rx.edge_start) and np.array_equal(tr.cnt_val, rx.cnt_val)
        # the suffix-order assembly on the real text: identical arrays
        from tests.helpers import assert_same_trie, suffix_order_np
        assert_same_trie(A.RadixTrie.from_suffix_order(tok, depth, *suffix_order_np(tok, depth + 1)), tr)


@pytest.mark.skipif(not os.path.exists(REF_CORPUS), reason="reference corpus not mounted")
def test_real_corpus_depth_32_anchors():
    """What the reference's own trainer log prints for its depth-32 radix trie of the same corpus
    (rnd/hotspot-curriculum/logs/d32-base-3SE_r1.log:5-6, :12-13, :17; rnd/sparsity-profile/README.md:97-101):
    radix nodes and edge chars, endpoint depths, count entries, the longest edge, chars on mass-1 edges, nodes of
    mass > 1, and the 65 root-child subtrees with their smallest and largest size.  Built with the product's level
    builder (bit-identical to the oracle's builders at depths 8 and 16 on the same text, and on synthetic corpora)."""
    import agpt_b200 as A
    tr = A.RadixTrie.build(_real_corpus_tokens(), 32)
    assert tr.radix_count - 1 == 1_666_214 and tr.total_edge_chars == 27_046_236
    assert tr.n_depth_files == 33 and tr.cnt_val.size == 2_780_616
    assert int(tr.edge_len[1:].max()) == 32
    mass1 = tr.edge_mass[1:] == 1
    assert int(tr.edge_len[1:][mass1].sum()) == 25_933_966
    assert int((~mass1).sum()) == 552_869
    assert int(tr.edge_len[1:][~mass1].sum()) == 1_112_270           # positions the reference's compact KV cache holds
    root_child = np.zeros(tr.radix_count, np.int64)
    for r in range(1, tr.radix_count):                               # ids are in breadth-first order: parents come first
        root_child[r] = r if tr.parent[r] == 0 else root_child[tr.parent[r]]
    sizes = np.bincount(root_child[1:])
    sizes = sizes[sizes > 0]
    assert sizes.size == 65 and sizes.min() == 1 and sizes.max() == 254_737 and sizes.sum() == 1_666_214


def test_golden_vectors_reproduce():
    path = os.path.join(os.path.dirname(__file__), "golden", "attention_small.npz")
    g = np.load(path)
    H, hd = int(g["H"]), int(g["hd"])
    out, w, w_off, _ = O.attn_fwd(g["parent"], H, hd, g["q"], g["k"], g["v"])
    dq, dk, dv = O.attn_bwd(g["parent"], H, hd, g["q"], g["k"], g["v"], w, w_off, g["dout"])
    for name, val in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
        assert rel_err(val, g[name]) < 1e-6, name
    gl = np.load(os.path.join(os.path.dirname(__file__), "golden", "loss_small.npz"))
    loss, grad = O.loss_per_query(gl["logits"], gl["q2n"], gl["qoff"], gl["radix_ids"], gl["token_ids"], gl["cnt_off"],
                                  gl["cnt_tok"], gl["cnt_val"], gl["mass_w"], float(gl["lam"]), float(gl["iw"]), False)
    assert rel_err(loss, gl["loss"]) < 1e-6 and rel_err(grad, gl["grad"]) < 1e-6


def test_model_oracle_agrees_with_an_independent_dense_model():
    """The whole-model restatement (per-node forward / backward of src/agpt/incremental_forward.cr and
    incremental_backward.cr with the ancestor accumulators) against a dense float64 autograd model that knows nothing
    of nodes, caches or accumulators -- only an ancestor mask: logits, loss and every weight gradient."""
    import agpt_b200 as A
    from agpt_b200 import model_file as MF
    from tests.helpers import model_oracle_step
    from tests.test_trainer_gpu import _reference
    corpus = A.synth_markov_corpus(260, 12, 2, 3)
    trie = A.RadixTrie.build(corpus, 6)
    parent, tokens, depth, radix_of = trie.char_tree()
    plan = A.WalkerPlan(parent, 64, -1)
    order = plan.dfs_to_node.astype(np.int64)
    p_dfs, tok, dep, rof = plan.parent_dfs.copy(), tokens[order], depth[order], radix_of[order]
    starts = np.concatenate([[True], rof[1:] != rof[:-1]])
    q2n = (np.cumsum(starts) - 1).astype(np.int32)
    qoff = np.concatenate([np.nonzero(starts)[0], [rof.size]]).astype(np.int32)
    rid = rof[starts].astype(np.int32)
    counts = (trie.cnt_off.astype(np.int32), trie.cnt_tok, trie.cnt_val)
    mw = A.mass_weights(trie.edge_mass[rid], np.diff(qoff), "linear")
    mf = MF.random_init(32, 2, 2, 12, 16, seed=1, std=0.2)
    unit = np.zeros(rof.size, np.int64)
    args = (mf, p_dfs, tok.astype(np.int32), dep, q2n, qoff, rid, counts, mw, 0.5, 0.7, None, unit)
    rl, rq, rg, rlog = _reference(*args)
    ol, oq, og, olog = model_oracle_step(*args)
    assert oq == rq and abs(ol - rl) / rl < 1e-5
    assert rel_err(olog, rlog) < 1e-5
    for k in rg:
        assert rel_err(og[k], rg[k], floor=1e-6) < 2e-5, k
