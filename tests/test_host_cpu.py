"""Host-side logic of the product library, checked on CPU: trie construction and ancestor indexing
bit-exact against the oracle's restatement of the reference builders, the on-disk radix directory
byte-for-byte, walker-plan invariants, the unit partitioner and the exported C symbols."""
import filecmp
import os
import re

import numpy as np
import pytest

import agpt_b200 as A
from agpt_b200 import _lib
from oracle import pyoracle as O
from tests.helpers import chain_tree, random_tree

TRIE_FIELDS = ("parent", "first_char_depth", "edge_len", "edge_mass", "endpoint_depth", "subtree_key", "edge_start",
               "edge_off", "edge_tok", "cnt_off", "cnt_tok", "cnt_val")


def _same_trie(tr, rx):
    assert tr.radix_count == rx.radix_count and tr.total_edge_chars == rx.total_edge_chars
    for name in TRIE_FIELDS:
        assert np.array_equal(getattr(tr, name), getattr(rx, name)), name


@pytest.mark.parametrize("n,vocab,order,depth,seed", [(20_000, 65, 2, 8, 0), (5_000, 96, 3, 12, 3), (300, 5, 1, 40, 9),
                                                      (2, 3, 1, 4, 1), (50, 2, 1, 64, 2)])
def test_trie_build_bit_exact(n, vocab, order, depth, seed):
    corpus = A.synth_markov_corpus(n, vocab, order, seed)
    tr = A.RadixTrie.build(corpus, depth)
    lv = O.Leveled(corpus, depth)
    rx = O.Radix(lv)
    _same_trie(tr, rx)
    assert tr.leveled_nodes == lv.n_nodes
    p1, t1, d1, r1 = tr.char_tree()
    p2, t2, d2 = rx.char_tree()
    assert np.array_equal(p1, p2) and np.array_equal(t1, t2) and np.array_equal(d1, d2)
    # ancestor index: walking the char tree's parents reproduces the trainer's ancestor lists
    for r in range(1, min(rx.radix_count, 400)):
        anc = rx.anc_ids[rx.anc_off[r]:rx.anc_off[r + 1]]
        walk, c = [], p1[rx.edge_start[r]]
        while c >= 0:
            walk.append(c)
            c = p1[c]
        assert walk[::-1] == list(anc)


def test_config1_trie_shape():
    """20k-char order-2 Markov corpus, depth 8: per-depth position counts of the synthetic stand-in."""
    corpus = A.synth_markov_corpus(20_000, 65, 2, 0)
    tr = A.RadixTrie.build(corpus, 8)
    _, _, depth, _ = tr.char_tree()
    assert tr.total_edge_chars == 65_985
    assert list(np.bincount(depth)[1:]) == [65, 1256, 3031, 5818, 9281, 12828, 15816, 17890]


@pytest.mark.parametrize("level,min_mass", [(1, 1), (2, 1), (1, 2), (2, 3)])
def test_trie_pruning_and_bigram_keys(level, min_mass):
    corpus = A.synth_markov_corpus(8_000, 30, 2, 5)
    tr = A.RadixTrie.build(corpus, 10, subtree_level=level, prune_min_mass=min_mass, prune_min_depth=4)
    rx = O.Radix(O.Leveled(corpus, 10), level, min_mass, 4)
    _same_trie(tr, rx)
    if min_mass > 1:
        deep = tr.first_char_depth[1:] >= 4
        assert (tr.edge_mass[1:][deep] >= min_mass).all()


def test_radix_dir_bytes_and_reload(tmp_path):
    corpus = A.synth_markov_corpus(6_000, 40, 2, 11)
    tr = A.RadixTrie.build(corpus, 9)
    rx = O.Radix(O.Leveled(corpus, 9))
    h = A.token_hash(corpus)
    assert h == O.token_hash(corpus)
    a, b = str(tmp_path / "product"), str(tmp_path / "oracle")
    tr.save_dir(a, corpus.size, 40, h, per_subtree=True)
    rx.write_dir(b, corpus.size, 40, h)
    names = sorted(f for f in os.listdir(b))
    assert names == sorted(f for f in os.listdir(a) if f not in ("manifest.bin", "subtrees"))
    for f in names:
        assert filecmp.cmp(os.path.join(a, f), os.path.join(b, f), shallow=False), f
    back = A.RadixTrie.load_dir(a)
    for name in TRIE_FIELDS:
        assert np.array_equal(getattr(back, name), getattr(tr, name)), name
    # per-subtree files: one per root child, sizes add up, manifest sorted by key
    subs = sorted(os.listdir(os.path.join(a, "subtrees")))
    assert len(subs) == int((tr.parent[1:] == 0).sum())
    raw = np.fromfile(os.path.join(a, "manifest.bin"), dtype=np.uint8)
    n_sub = int(np.frombuffer(raw[8:12].tobytes(), np.int32)[0])
    assert n_sub == len(subs)
    with pytest.raises(A.AgptError):
        A.RadixTrie.load_dir(str(tmp_path / "missing"))


@pytest.mark.parametrize("level", [1, 2])
def test_subtree_files_bytes_and_reload(tmp_path, level):
    """subtrees/*.bin and manifest.bin byte for byte against the oracle's writer (unigram and bigram keys), and
    each file read back as a trie of its own: local ids in file order, parents remapped (a parent outside the file
    becomes the local root), edges, counts and char positions as the reference's load_subtree lays them out
    (src/cuda/agpt_train.cu:495-669)."""
    corpus = A.synth_markov_corpus(5_000, 30, 2, 7)
    tr = A.RadixTrie.build(corpus, 9, subtree_level=level)
    rx = O.Radix(O.Leveled(corpus, 9), level)
    a, b = str(tmp_path / "product"), str(tmp_path / "oracle")
    tr.save_dir(a, corpus.size, 30, A.token_hash(corpus), per_subtree=True)
    os.makedirs(b)
    rx.write_subtree_files(b)
    assert filecmp.cmp(os.path.join(a, "manifest.bin"), os.path.join(b, "manifest.bin"), shallow=False)
    names = sorted(os.listdir(os.path.join(b, "subtrees")))
    assert names == sorted(os.listdir(os.path.join(a, "subtrees"))) and len(names) > 10
    for f in names:
        assert filecmp.cmp(os.path.join(a, "subtrees", f), os.path.join(b, "subtrees", f), shallow=False), f
    keys, nodes, chars, ep = A.RadixTrie.manifest(a)
    assert np.array_equal(keys, np.unique(tr.subtree_key[1:])) and nodes.sum() == tr.radix_count - 1
    assert chars.sum() == tr.total_edge_chars
    for key, nn, ch, me in zip(keys, nodes, chars, ep):
        sub = A.RadixTrie.load_subtree(a, int(key))
        ids = np.nonzero(tr.subtree_key == key)[0]
        ids = ids[ids > 0]                                   # global ids in emission (= file) order
        assert sub.radix_count == nn + 1 == ids.size + 1 and sub.total_edge_chars == ch
        assert int(tr.endpoint_depth[ids].max()) == me
        local = {int(g): i + 1 for i, g in enumerate(ids)}
        assert np.array_equal(sub.parent[1:], [local.get(int(tr.parent[g]), 0) for g in ids])
        for name in ("first_char_depth", "edge_len", "edge_mass", "endpoint_depth"):
            assert np.array_equal(getattr(sub, name)[1:], getattr(tr, name)[ids]), name
        assert np.array_equal(sub.edge_start[1:], np.concatenate([[0], np.cumsum(tr.edge_len[ids])[:-1]]))
        assert np.array_equal(sub.edge_tok, np.concatenate([tr.edge_tok[tr.edge_off[g]:tr.edge_off[g + 1]] for g in ids]))
        assert np.array_equal(sub.cnt_val, np.concatenate([tr.cnt_val[tr.cnt_off[g]:tr.cnt_off[g + 1]] for g in ids]))
        assert np.array_equal(np.diff(sub.cnt_off)[1:], np.diff(tr.cnt_off)[ids])
    with pytest.raises(A.AgptError):
        A.RadixTrie.load_subtree(a, 999_999)


def _brute_plan_check(parent, tile_m):
    plan = A.WalkerPlan(parent, tile_m, -1)
    n = parent.size
    d2n, n2d = plan.dfs_to_node, plan.node_to_dfs
    assert sorted(d2n) == list(range(n)) and np.array_equal(n2d[d2n], np.arange(n))
    depth = O.tree_depth_fast(parent)
    assert np.array_equal(plan.depth, depth[d2n])
    # parent links survive the relabelling and every parent precedes its children
    pp = plan.parent_dfs
    assert np.array_equal(np.where(pp < 0, -1, d2n[np.maximum(pp, 0)]), parent[d2n])
    assert (pp < np.arange(n)).all()
    # interval property: a is an ancestor-or-self of i  <=>  a <= i < sub_end[a]
    anc = np.zeros((n, n), bool)
    for i in range(n):
        c = i
        while c >= 0:
            anc[c, i] = True
            c = pp[c]
    idx = np.arange(n)
    interval = (idx[:, None] <= idx[None, :]) & (idx[None, :] < plan.sub_end[:, None])
    assert np.array_equal(anc, interval)
    assert plan.sum_depth == int(depth.sum())
    kids = np.bincount(parent[parent >= 0], minlength=n)
    assert plan.sum_group_prefix == int(depth[kids > 0].sum())
    assert plan.n_groups == int((kids > 0).sum()) + 1
    assert plan.chain_rows == int(sum(plan.depth[t * tile_m] - 1 for t in range(plan.n_tiles)))
    return plan


@pytest.mark.parametrize("n,md,seed,tile", [(1, 1, 0, 32), (37, 5, 1, 32), (300, 9, 2, 64), (257, 30, 3, 128), (129, 129, 4, 64)])
def test_plan_invariants(n, md, seed, tile):
    parent = chain_tree(n) if md >= n else random_tree(n, md, seed, roots=min(3, n))
    _brute_plan_check(parent, tile)


def test_plan_accepts_any_id_order_and_rejects_cycles():
    parent = random_tree(200, 8, 5)
    perm = np.random.default_rng(0).permutation(200)
    inv = np.argsort(perm)
    shuffled = np.where(parent[perm] < 0, -1, inv[np.maximum(parent[perm], 0)]).astype(np.int32)
    _brute_plan_check(shuffled, 64)
    bad = parent.copy()
    bad[10], bad[20] = 20, 10
    with pytest.raises(A.AgptError):
        A.WalkerPlan(bad, 64, -1)
    with pytest.raises(A.AgptError):
        A.WalkerPlan(np.array([5], np.int32), 64, -1)
    with pytest.raises(A.AgptError):
        A.WalkerPlan(parent, 48, -1)


def test_units_and_partition():
    parent = random_tree(3000, 10, 7, roots=9)
    plan = A.WalkerPlan(parent, 64, -1)
    b1, e1 = plan.units(1)
    assert b1[0] == 0 and e1[-1] == plan.n and np.array_equal(b1[1:], e1[:-1])
    assert (plan.depth[b1] == 1).all() and len(b1) == 9
    b2, e2 = plan.units(2)
    assert b2[0] == 0 and e2[-1] == plan.n and np.array_equal(b2[1:], e2[:-1])
    assert set(plan.depth[b2]) <= {1, 2}
    w = e2 - b2
    owner = A.partition_lpt(w, 4)
    loads = np.bincount(owner, weights=w, minlength=4)
    assert loads.max() <= w.sum() / 4 + w.max()
    # shards cover every node exactly once (context rows aside) and keep chains intact
    seen = np.zeros(plan.n, int)
    for r in range(4):
        lp, ids, ctx = A.shard_tree(parent, r, 4, level=2)
        seen[ids[~ctx]] += 1
        depth_local = O.tree_depth_fast(lp) if lp.size else lp
        assert np.array_equal(depth_local, O.tree_depth_fast(parent)[ids])
    assert (seen == 1).all()


def test_every_declared_symbol_is_exported():
    hdr = open(os.path.join(os.path.dirname(__file__), "..", "include", "agpt_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    names = set(re.findall(r"\b((?:agpt_b200|cuda)_[a-zA-Z0-9_]+)\s*\(", hdr))
    assert len(names) >= 30
    L = _lib.lib()
    for name in sorted(names):
        assert hasattr(L, name), name
    assert names == set(_lib.SIGNATURES), names ^ set(_lib.SIGNATURES)
    assert b"sm_100a" in L.agpt_b200_version()


def test_compute_entry_points_refuse_without_a_device_plan():
    """No CPU fallback: a plan without device index arrays is rejected by the kernels' launchers."""
    plan = A.WalkerPlan(chain_tree(10), 64, -1)
    rc = _lib.lib().agpt_b200_attn_fwd(plan._h, 1, 1, 1, 0, 1, 1, 2, 16, 0.25, None)
    assert rc == -1 and b"device" in _lib.lib().agpt_b200_last_error()
    assert plan.workspace_bytes(64) >= 256


def test_mass_weights_match_oracle():
    rng = np.random.default_rng(3)
    em = rng.integers(1, 5000, size=50)
    el = rng.integers(1, 9, size=50)
    for mode, code in (("log", 1), ("sqrt", 2), ("linear", 3), ("off", 0)):
        assert np.allclose(A.mass_weights(em, el, mode), O.mass_weights(em, el, code), rtol=1e-6, atol=0)


def test_rope_table_matches_oracle():
    for hd in (16, 32, 64):
        c, s = A.rope_table(128, hd)
        co, so = O.rope_table(128, hd)
        assert np.array_equal(c, co) and np.array_equal(s, so)


@pytest.mark.parametrize("vocab,order,n,depth", [(2, 1, 40, 6), (3, 1, 200, 8), (4, 2, 500, 5), (12, 2, 1500, 8), (65, 3, 3000, 16),
                                                   (5, 1, 64, 30), (2, 1, 12, 10), (96, 4, 2500, 40)])
def test_trie_from_suffix_order_equals_level_builder(vocab, order, n, depth):
    """The linear assembly from a suffix order reproduces the level-by-level builder array for array: ids, edges,
    masses, counts, keys, char positions; unigram and bigram keys; with and without pruning; small alphabets and deep
    tries make many suffixes run into the end of the corpus."""
    from tests.helpers import assert_same_trie, suffix_order
    for seed in range(4):
        corpus = A.synth_markov_corpus(n, vocab, order, seed)
        sa, lcp = suffix_order(corpus, depth + 1)
        for level, mass, mdepth in ((1, 1, 4), (2, 1, 4), (1, 2, 2), (2, 3, 1), (1, 2, 4)):
            want = A.RadixTrie.build(corpus, depth, subtree_level=level, prune_min_mass=mass, prune_min_depth=mdepth)
            got = A.RadixTrie.from_suffix_order(corpus, depth, sa, lcp, subtree_level=level, prune_min_mass=mass,
                                                prune_min_depth=mdepth)
            assert_same_trie(got, want)


def test_trie_from_suffix_order_rejects_short_corpus():
    corpus = A.synth_markov_corpus(8, 3, 1, 0)
    with pytest.raises(A.AgptError):
        A.RadixTrie.from_suffix_order(corpus, 8, np.arange(7, dtype=np.int32), np.zeros(7, np.int32))


@pytest.mark.parametrize("sampler", [1, 2, 3, 4])
def test_lightning_sampler_matches_oracle(sampler):
    """Sampled node sets, ancestor counts, masses and the generator state against the restatement, bit for bit, over
    several super-epochs that continue one generator stream (with and without the mass cap)."""
    corpus = A.synth_markov_corpus(4000, 20, 2, 7)
    trie = A.RadixTrie.build(corpus, 10)
    for max_mass in (0, 40):
        state = 0x5c115e1
        want_state = state
        for _ in range(3):
            rs, na, off, mass, nodes, state = trie.lightning_sample(sampler, 9, state, p_stop=0.3, max_mass=max_mass)
            want, want_state = O.lightning_sample(trie.parent, trie.edge_mass, trie.first_char_depth, trie.edge_len, sampler, 9,
                                                  want_state, 0.3, max_mass)
            assert state == want_state
            for i, (pick, n_anc, m, ids) in enumerate(want):
                assert (int(rs[i]), int(na[i])) == (pick, n_anc) and mass[i] == m
                assert nodes[off[i]:off[i + 1]].tolist() == ids
                if sampler != 4:      # the set is closed under "parent" up to the root and holds the whole subtree of the pick
                    assert set(int(trie.parent[x]) for x in ids) <= set(ids) | {0}


def test_lr_schedule_matches_oracle():
    for sched, code in (("constant", 0), ("cosine", 1), ("warmup-cosine", 2)):
        for total, warm in ((1, 0), (10, 3), (130, 13), (5, 9)):
            for step in range(0, total + 3):
                got, want = A.compute_lr(3e-4, step, total, warm, sched), float(O.compute_lr(3e-4, step, total, warm, code))
                assert abs(got - want) <= 1e-6 * 3e-4, (sched, total, warm, step)
    assert A.compute_lr(1.0, 0, 100, 10, "warmup-cosine") == pytest.approx(0.1) and A.compute_lr(1.0, 100, 100, 10, "cosine") == pytest.approx(0.0, abs=1e-7)


def test_units_capped_partition_all_rows():
    """Capped units tile the depth-first order exactly; a unit over the cap can only be a bare chain; without a
    cap they are the plain units."""
    corpus = A.synth_markov_corpus(5000, 12, 2, 1)
    parent = A.RadixTrie.build(corpus, 9).char_tree()[0]
    plan = A.WalkerPlan(parent, 64, -1)
    for level in (1, 2):
        ub, ue = plan.units(level)
        b, e = plan.units_capped(level, 10 ** 9)
        assert np.array_equal(b, ub) and np.array_equal(e, ue)
        for cap in (10, 100, 1000):
            b, e = plan.units_capped(level, cap)
            assert b[0] == 0 and e[-1] == plan.n and np.array_equal(b[1:], e[:-1])
            for bb, ee in zip(b, e):
                whole = plan.sub_end[bb] == ee
                chain = all(plan.sub_end[j] == plan.sub_end[bb] for j in range(bb, ee))
                assert whole or chain                       # a subtree, or the unary top of one
                assert ee - bb <= cap or chain


def test_build_gpu_on_a_tiny_corpus_uses_the_level_builder():
    from tests.helpers import assert_same_trie
    corpus = A.synth_markov_corpus(9, 3, 1, 2)
    assert_same_trie(A.RadixTrie.build_gpu(corpus, 12), A.RadixTrie.build(corpus, 12))


@pytest.mark.parametrize("builder", ["level", "suffix_order"])
def test_radix_trie_is_lossless_against_brute_force_counts(builder):
    """The check of the reference's src/tools/radix_verify.cr:58-106 with the leveled trie replaced by brute force:
    every radix node's root path is a prefix that occurs in the corpus, its counts are exactly the next-token
    counts after the occurrences of that path, its edge mass is the number of occurrences of the path up to its
    first edge character that continue, and every prefix with two or more continuations is some node's endpoint."""
    from collections import Counter, defaultdict
    from tests.helpers import suffix_order
    depth = 6
    corpus = A.synth_markov_corpus(1200, 6, 2, 4)
    c = corpus.tolist()
    n = len(c)
    nxt = defaultdict(Counter)                 # prefix -> Counter(next token); starts 0 .. n-2 as the builders use
    for s0 in range(n - 1):
        for d in range(1, depth + 1):
            if s0 + d - 1 > n - 1:
                break
            key = tuple(c[s0:s0 + d])
            nxt[key]                           # the prefix exists even if nothing follows it
            if s0 + d <= n - 1:
                nxt[key][c[s0 + d]] += 1
    if builder == "level":
        t = A.RadixTrie.build(corpus, depth)
    else:
        t = A.RadixTrie.from_suffix_order(corpus, depth, *suffix_order(corpus, depth + 1))
    endpoints = set()
    for r in range(1, t.radix_count):
        path, cur = [], r
        while cur != 0:
            path = t.edge_tok[t.edge_off[cur]:t.edge_off[cur + 1]].tolist() + path
            cur = int(t.parent[cur])
        key = tuple(path)
        assert key in nxt and len(key) == t.endpoint_depth[r]
        got = dict(zip(t.cnt_tok[t.cnt_off[r]:t.cnt_off[r + 1]].tolist(), t.cnt_val[t.cnt_off[r]:t.cnt_off[r + 1]].tolist()))
        assert got == dict(nxt[key])
        first = key[:t.first_char_depth[r]]
        assert t.edge_mass[r] == sum(nxt[first].values())
        endpoints.add(key)
    for key, cnt in nxt.items():
        if len(cnt) >= 2 or (len(key) == depth and len(cnt) >= 1):
            assert key in endpoints
    assert len(endpoints) == t.radix_count - 1


def test_lightning_lr_weights_match_oracle():
    from agpt_b200 import trainer as T
    masses = [729.0, 1272.0, 3.0, 0.0, 88000.0]
    for mode, code in (("off", 0), ("log", 1), ("sqrt", 2), ("linear", 3)):
        got, want = T.lightning_lr_weights(masses, mode), O.lightning_lr_weights(masses, code)
        assert np.allclose(got, want, rtol=1e-15, atol=0)
        assert mode == "off" or abs(float(np.mean(got)) - 1.0) < 1e-12
    assert T.lightning_lr_weights([], "log").size == 0 and np.array_equal(T.lightning_lr_weights([0.0, 0.0], "linear"), [0.0, 0.0])


def test_attention_wrappers_refuse_mismatched_tensors_before_any_launch():
    """The C entry points take no row count, so the Python wrappers must refuse every tensor whose shape, dtype,
    layout or device differs from what the plan needs -- checked here on CPU tensors through the same validator
    (require_cuda=False) that attn_forward / attn_backward / attn_backward_static call first."""
    import torch
    plan = A.WalkerPlan(random_tree(100, 5, 1), 64, -1)
    H, D = 2, 64
    ok = lambda rows=100, cols=D, dt=torch.float32: torch.zeros((rows, cols), dtype=dt)   # noqa: E731
    lse = torch.zeros((100, H))
    good = dict(f32_rows=[("q", ok()), ("out", ok()), ("dout", ok()), ("dq", ok()), ("dk", ok()), ("dv", ok())],
                kv_rows=[("k", ok()), ("v", ok())], lse=lse)
    assert A.validate_attn_args(plan, H, **good, require_cuda=False) == (64, 32)
    assert A.validate_attn_args(plan, H, [("q", ok())], [("k", ok(dt=torch.bfloat16)), ("v", ok(dt=torch.bfloat16))], lse,
                                require_cuda=False) == (64, 32)

    def bad(match, **kw):
        args = dict(good)
        args.update(kw)
        with pytest.raises(A.AgptError, match=match):
            A.validate_attn_args(plan, H, **args, require_cuda=False)

    bad("shape", f32_rows=[("q", ok(rows=99))])                                  # fewer rows than the plan
    bad("shape", f32_rows=[("q", ok()), ("dq", ok(rows=64))])                    # a short output tensor
    bad("shape", f32_rows=[("q", ok()), ("dout", ok(cols=32))])
    bad("shape", kv_rows=[("k", ok(rows=50)), ("v", ok())])
    bad("shape", lse=torch.zeros((100, 4)))
    bad("shape", lse=torch.zeros((99, H)))
    bad("dtype", f32_rows=[("q", ok()), ("dk", ok(dt=torch.float64))])
    bad("dtype", kv_rows=[("k", ok(dt=torch.float16)), ("v", ok())])
    bad("same dtype", kv_rows=[("k", ok(dt=torch.bfloat16)), ("v", ok())])
    bad("dtype", lse=torch.zeros((100, H), dtype=torch.float64))
    bad("contiguous", f32_rows=[("q", ok()), ("dv", torch.zeros((D, 100)).t())])
    bad("contiguous", kv_rows=[("k", torch.zeros((100, 2 * D))[:, ::2]), ("v", ok())])
    with pytest.raises(A.AgptError, match="multiple"):
        A.validate_attn_args(plan, 3, [("q", ok())], require_cuda=False)
    with pytest.raises(A.AgptError, match="head_dim"):
        A.validate_attn_args(plan, 8, [("q", ok())], require_cuda=False)         # head_dim 8
    with pytest.raises(A.AgptError, match="CUDA"):
        A.validate_attn_args(plan, H, **good)                                    # CPU tensors where device tensors are required


@pytest.mark.parametrize("sampler", [1, 3])
def test_lightning_unit_trains_its_ancestors_and_counts_them_in_the_mass_mean(sampler):
    """The reference's lightning samplers prepend the sampled node's ancestors, and the code that runs trains them
    like every other position: the mass-weight mean of the chunk runs over all its queries, ancestors included
    (src/cuda/agpt_train.cu:4601-4637).  The launch group of a sampled unit must therefore carry no untrained rows and
    its mass weights must equal the oracle's restatement over every row of the unit."""
    import torch
    from agpt_b200 import trainer as T
    corpus = A.synth_markov_corpus(900, 12, 2, 13)
    trie = A.RadixTrie.build(corpus, 7)
    space = T.SampleSpace(trie)
    rs, na, off, _, nodes, _ = trie.lightning_sample(sampler, 6, 0x5c115e1, p_stop=0.4)
    with_ancestors = 0
    for s in range(6):
        ids = nodes[off[s]:off[s + 1]]
        with_ancestors += int(trie.parent[rs[s]] > 0)
        g = space.group(ids, [], "linear", 16, torch.device("cpu"))
        assert g.trained is None and g.n_trained_rows == g.n == int(trie.edge_len[ids].sum())
        rid = g.rid.numpy()
        assert sorted(rid.tolist()) == sorted(np.asarray(ids).tolist())          # one loss node per sampled radix node
        want = O.mass_weights(trie.edge_mass[rid], np.diff(g.qoff.numpy()), 3)  # mean over all queries of the unit
        assert np.allclose(g.mass_w.numpy(), want, rtol=1e-6, atol=0)
    assert with_ancestors > 0


def test_build_pins_the_cutlass_release(tmp_path, monkeypatch):
    """The GEMM sources re-instantiate a CUTLASS collective through its type aliases, so the build takes header trees of
    the pinned release only: another release inside a package is passed over, one named explicitly is refused."""
    from agpt_b200 import build as B
    inc = tmp_path / "include" / "cutlass"
    (inc / "gemm" / "device").mkdir(parents=True)
    (inc / "gemm" / "device" / "gemm_universal.h").write_text("")
    (inc / "version.h").write_text("#define CUTLASS_MAJOR 3\n#define CUTLASS_MINOR 9\n#define CUTLASS_PATCH 2\n")
    assert B.cutlass_version(str(tmp_path / "include")) == (3, 9, 2)
    assert B.cutlass_version(str(tmp_path)) is None
    monkeypatch.setenv("AGPT_CUTLASS_INCLUDE", str(tmp_path / "include"))
    with pytest.raises(RuntimeError, match="needed"):
        B.cutlass_include()
    (inc / "version.h").write_text("#define CUTLASS_MAJOR %d\n#define CUTLASS_MINOR %d\n#define CUTLASS_PATCH 7\n" % B.CUTLASS_PINNED)
    assert B.cutlass_include() == str(tmp_path / "include")
    monkeypatch.delenv("AGPT_CUTLASS_INCLUDE")
    found = B.cutlass_include()
    assert found is None or B.cutlass_version(found)[:2] == B.CUTLASS_PINNED


def test_launch_groups_keep_units_consecutive_and_count_them_by_offsets():
    """Rows of a unit are consecutive in a launch group, so the trainer counts a unit's trained queries as the difference of
    a running sum at the unit offsets; that must equal the scattered count over unit_of_row, whatever the packing."""
    import torch
    from agpt_b200 import trainer as T
    corpus = A.synth_markov_corpus(6000, 20, 2, 5)
    trie = A.RadixTrie.build(corpus, 9)
    for group_rows, cap in ((700, None), (2500, 900), (10**9, None)):
        groups, total = T.build_groups(trie, 0, 1, group_rows, "linear", 16, torch.device("cpu"), level=2, unit_cap=cap)
        assert sum(g.n for g in groups) >= total
        for g in groups:
            assert g.unit_off is not None and g.unit_off.numel() == g.n_units + 1
            u = g.unit_of_row.numpy()
            assert np.all(np.diff(u) >= 0) and int(g.unit_off[-1]) == g.n
            pos = torch.from_numpy(np.random.default_rng(g.n).random(g.n) < 0.6)
            run = torch.nn.functional.pad(torch.cumsum(pos, 0, dtype=torch.int32), (1, 0))
            got = (run[g.unit_off[1:]] - run[g.unit_off[:-1]]).to(torch.float32)
            want = torch.zeros(g.n_units).index_add_(0, g.unit_of_row, pos.to(torch.float32))
            assert torch.equal(got, want)


def _py_markov(n, vocab, order, seed, repeat_log2=0):
    """Plain-Python restatement of the synthetic corpus generator (splitmix64 stream, Zipf(1.1) slots and symbols,
    optional injected repeats), for small n."""
    M64 = (1 << 64) - 1

    def sm(x):
        x = (x + 0x9E3779B97F4A7C15) & M64
        z = x
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
        return z ^ (z >> 31)

    def cdf(k):
        w = np.cumsum([(r + 1) ** -1.1 for r in range(k)])
        w = w / w[-1]
        w[-1] = 1.0
        return w

    def inv(c, u):
        lo, hi = 0, len(c) - 1
        while lo < hi:
            mid = (lo + hi) // 2
            if u < c[mid]:
                hi = mid
            else:
                lo = mid + 1
        return lo

    zipf, slot = cdf(vocab), cdf(6)
    # the library accumulates the weights in double precision one by one, as np.cumsum does
    modulus = vocab ** order
    ctx, s = 0, sm(seed)
    out = []
    i = 0
    while i < n:
        if repeat_log2 > 0 and i > 0:
            s = sm(s)
            if (s >> (64 - repeat_log2)) == 0:
                s = sm(s)
                ln = 64 + s % 193
                s = sm(s)
                src = s % i
                t = 0
                while t < ln and i + t < n:
                    sym = out[src + t]
                    out.append(sym)
                    ctx = (ctx * vocab + sym) % modulus
                    t += 1
                i += t
                continue
        h = sm(seed ^ ((ctx * 0x9E3779B97F4A7C15) & M64))
        s = sm(s)
        j = inv(slot, (s >> 11) * (1.0 / 9007199254740992.0))
        sym = 0
        for _ in range(j + 1):
            h = sm(h)
            sym = inv(zipf, (h >> 11) * (1.0 / 9007199254740992.0))
        out.append(sym)
        ctx = (ctx * vocab + sym) % modulus
        i += 1
    return np.asarray(out, np.int32)


def test_synthetic_corpus_generators_match_their_restatement():
    for n, vocab, order, seed, rep in [(3000, 12, 2, 5, 0), (4000, 12, 2, 5, 6), (2500, 96, 4, 0, 5), (700, 65, 3, 1, 1)]:
        got = A.synth_markov_corpus(n, vocab, order, seed, rep)
        assert np.array_equal(got, _py_markov(n, vocab, order, seed, rep)), (n, vocab, order, seed, rep)


def test_injected_repeats_make_the_pruned_trie_deep():
    """A plain low-order Markov source has no long verbatim repeats, so after count<2 pruning its trie stays shallow
    whatever the depth cap; with injected repeats it reaches the cap (depth 128, the deep configuration's shape)."""
    # pruning from depth 1 here: in a 20k-char corpus rare trigrams occur once, and edges that start above the
    # pruning depth are kept whatever their count (in the 20M-char configuration every short prefix is frequent)
    plain = A.RadixTrie.build(A.synth_markov_corpus(20_000, 12, 2, 3), 128, 1, 2, 1)
    deep = A.RadixTrie.build(A.synth_markov_corpus(20_000, 12, 2, 3, 6), 128, 1, 2, 1)
    d_plain = int(plain.char_tree()[2].max())
    d_deep = int(deep.char_tree()[2].max())
    assert d_plain < 40 and d_deep == 128
