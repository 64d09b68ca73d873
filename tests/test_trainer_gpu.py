"""The trie-walk trainer (embedding -> layers -> logits -> loss -> backward) against a dense float64 torch
model on CPU that uses an explicit ancestor mask, the oracle's RoPE tables and the oracle's loss."""
import numpy as np
import pytest

import agpt_b200 as A
from agpt_b200 import model_file as MF
from agpt_b200 import trainer as T
from oracle import pyoracle as O
from tests.helpers import TOL_BF16, TOL_F32, rel_err

pytestmark = pytest.mark.gpu


def _reference(mf, parent, tokens, depth, q2n, qoff, rid, counts, mass_w, lam, iw, trained, unit_of_row):
    """Dense reference: float64 torch autograd, mask[i, a] = a is an ancestor-or-self of i."""
    import torch
    import torch.nn.functional as F
    n, D, H = parent.size, mf.d_model, mf.n_heads
    hd = D // H
    P = {k: torch.from_numpy(v.astype(np.float64)).requires_grad_(True) for k, v in mf.mats}
    mask = np.zeros((n, n), bool)
    for i in range(n):
        c = i
        while c >= 0:
            mask[i, c] = True
            c = parent[c]
    mask = torch.from_numpy(mask)
    cos, sin = O.rope_table(mf.seq_len, hd)
    pos = np.minimum(depth - 1, mf.seq_len - 1)
    c = torch.from_numpy(cos[pos].astype(np.float64))[:, None, :]      # [n, 1, hd]
    s = torch.from_numpy(sin[pos].astype(np.float64))[:, None, :]

    def rope(x):
        x = x.view(n, H, hd)
        x0, x1 = x[..., 0::2], x[..., 1::2]
        cc, ss = c[..., 0::2], s[..., 0::2]
        out = torch.stack([x0 * cc - x1 * ss, x0 * ss + x1 * cc], dim=-1)
        return out.reshape(n, H, hd)

    x = P["token_emb"][torch.from_numpy(tokens.astype(np.int64))]
    for l in range(mf.n_layers):
        g = lambda name: P[f"layer{l}.{name}"]  # noqa: E731
        x1 = F.layer_norm(x, (D,), g("ln1.gamma")[0], g("ln1.beta")[0], 1e-5)
        q = rope(x1 @ g("wq.w") + g("wq.b"))
        k = rope(x1 @ g("wk.w") + g("wk.b"))
        v = (x1 @ g("wv.w") + g("wv.b")).view(n, H, hd)
        sc = torch.einsum("ihd,jhd->hij", q, k) / np.sqrt(hd)
        sc = sc.masked_fill(~mask[None], float("-inf"))
        a = torch.einsum("hij,jhd->ihd", torch.softmax(sc, dim=-1), v).reshape(n, D)
        x = x + a @ g("wo.w") + g("wo.b")
        x2 = F.layer_norm(x, (D,), g("ln2.gamma")[0], g("ln2.beta")[0], 1e-5)
        x = x + F.relu(x2 @ g("l1.w") + g("l1.b")) @ g("l2.w") + g("l2.b")
    xf = F.layer_norm(x, (D,), P["final.gamma"][0], P["final.beta"][0], 1e-5)
    logits = xf @ P["out.w"] + P["out.b"]
    loss, dlog = O.loss_per_query(logits.detach().numpy().astype(np.float32), q2n, qoff, rid, tokens, *counts, mass_w, lam, iw)
    if trained is not None:
        loss = loss * trained
        dlog = dlog * trained[:, None]
    n_tr = int((loss > 0).sum())
    per_unit = np.bincount(unit_of_row, weights=(loss > 0).astype(np.float64), minlength=int(unit_of_row.max()) + 1)
    scale = np.where(per_unit > 0, 1.0 / np.maximum(per_unit, 1), 0.0)[unit_of_row]      # per-unit 1 / trained queries
    logits.backward(torch.from_numpy(dlog.astype(np.float64) * scale[:, None]))
    return float(loss[loss > 0].sum()), n_tr, {k: v.grad.numpy() for k, v in P.items()}, logits.detach().numpy()


@pytest.mark.parametrize("world,bf16,unit_cap,vocab", [(1, False, None, 12), (2, False, None, 12), (1, True, None, 12), (2, False, 40, 12),
                                                       (1, False, None, 13)])
def test_group_step_matches_dense_reference(cuda, world, bf16, unit_cap, vocab):
    """vocab 13: a vocabulary that is not a multiple of 4 (like the reference's 65) takes the padded logits projection."""
    import torch
    corpus = A.synth_markov_corpus(700, vocab, 2, 3)
    trie = A.RadixTrie.build(corpus, 7, subtree_level=1 if world == 1 else 2)
    mf = MF.random_init(32, 2, 2, vocab, 16, seed=1, std=0.2)
    counts_np = (trie.cnt_off.astype(np.int32), trie.cnt_tok, trie.cnt_val)
    counts = [torch.from_numpy(np.ascontiguousarray(c)).to(cuda) for c in counts_np]
    lam, iw = 0.5, 0.7
    grads, loss_sum, n_q, ref_grads, ref_loss, ref_q = None, 0.0, 0, None, 0.0, 0
    for rank in range(world):
        groups, total = T.build_groups(trie, rank, world, 500, "linear", mf.seq_len, cuda, unit_cap=unit_cap)
        if unit_cap:     # units cut below the bigram level carry context chains longer than one row
            assert any(g.trained is not None and int((g.trained == 0).sum()) > g.n_units for g in groups)
        model = T.TrieWalkModel(mf, cuda)
        for p in model.parameters():
            p.grad = torch.zeros_like(p)
        for g in groups:
            ls, nq = model.group_step(g, counts, entropy_lambda=lam, intermediate_weight=iw, bf16_store=bf16)
            loss_sum += ls
            n_q += nq
            tr = None if g.trained is None else g.trained.cpu().numpy()
            rl, rq, rg, _ = _reference(mf, g.plan.parent_dfs.copy(), g.tokens32.cpu().numpy(), g.plan.depth.copy(),
                                       g.q2n.cpu().numpy(), g.qoff.cpu().numpy(), g.rid.cpu().numpy(), counts_np,
                                       None if g.mass_w is None else g.mass_w.cpu().numpy(), lam, iw, tr,
                                       g.unit_of_row.cpu().numpy())
            ref_loss += rl
            ref_q += rq
            ref_grads = rg if ref_grads is None else {k: ref_grads[k] + rg[k] for k in rg}
        got = {k: v.grad.cpu().numpy().astype(np.float64) for k, v in model.params.items()}
        grads = got if grads is None else {k: grads[k] + got[k] for k in got}
    assert n_q == ref_q == trie.total_edge_chars - int((np.diff(trie.cnt_off)[1:] == 0).sum()) or n_q == ref_q
    tol = TOL_BF16 if bf16 else TOL_F32
    assert abs(loss_sum - ref_loss) / ref_loss < tol
    for k in ref_grads:
        assert rel_err(grads[k], ref_grads[k], floor=1e-6) < tol, k


def test_training_lowers_loss_and_round_trips_model(cuda, tmp_path):
    import torch
    corpus = A.synth_markov_corpus(3000, 20, 2, 5)
    trie = A.RadixTrie.build(corpus, 8)
    d = str(tmp_path / "trie")
    trie.save_dir(d, corpus.size, 20, A.token_hash(corpus))
    mf = MF.random_init(32, 2, 2, 20, 16, seed=2)
    mp = str(tmp_path / "m.model")
    MF.save(mp, mf)
    out = str(tmp_path / "out.model")
    lines = []
    import builtins
    real_print = builtins.print
    builtins.print = lambda *a, **k: (lines.append(" ".join(str(x) for x in a)), real_print(*a, **k))
    try:
        T.main(["--model", mp, "--trie-dir", d, "--epochs", "10", "--lr", "0.01", "--optimizer", "adam", "--no-accumulate",
                "--group-rows", "4000", "--mass-weight", "log", "--save", out])
    finally:
        builtins.print = real_print
    ep = [ln for ln in lines if ln.startswith("Epoch ")]
    assert len(ep) == 10
    losses = [float(ln.split("loss=")[1].split()[0]) for ln in ep]
    assert losses[-1] < 0.9 * losses[0] and all(np.isfinite(losses))
    new = MF.load(out)
    changed = [n for (n, a), (_, b) in zip(mf.mats, new.mats) if not np.array_equal(a, b)]
    assert len(changed) == len(mf.mats)          # every weight matrix moved (the reference's own fundamentals test)
    del torch


@pytest.mark.parametrize("name", ["sgd", "momentum", "rmsprop", "adam"])
def test_flat_optimizer_matches_torch(cuda, name):
    """Two accumulated epochs with the library's fused step move the weights as torch's optimizer of the same
    rule does from the same gradients (1e-5 of the largest weight)."""
    import torch
    corpus = A.synth_markov_corpus(600, 12, 2, 9)
    trie = A.RadixTrie.build(corpus, 6)
    mf = MF.random_init(32, 2, 1, 12, 16, seed=4, std=0.2)
    counts = [torch.from_numpy(np.ascontiguousarray(c)).to(cuda) for c in (trie.cnt_off.astype(np.int32), trie.cnt_tok, trie.cnt_val)]
    groups, _ = T.build_groups(trie, 0, 1, 100000, "off", mf.seq_len, cuda)
    model = T.TrieWalkModel(mf, cuda)
    opt = T.make_optimizer(name, model, 1e-2)
    assert isinstance(opt, T.FlatOptimizer)
    shadow = [p.detach().clone().requires_grad_(True) for p in model.parameters()]
    topt = T.make_optimizer(name, shadow, 1e-2)
    for _ in range(2):
        model.bind_grads()
        opt.zero_grad()
        for g in groups:
            model.group_step(g, counts)
        for sp, p in zip(shadow, model.parameters()):
            sp.grad = p.grad.clone()
        opt.step()
        topt.step()
        assert float(model.flat_grad[:model.n_flat].abs().max()) == 0.0
        for sp, p in zip(shadow, model.parameters()):
            assert float((sp - p).abs().max()) < 1e-5 * max(1.0, float(p.abs().max()))


def test_gradients_do_not_depend_on_packing_or_rank_count(cuda):
    """Same bigram units, packed into launches of different sizes and spread over 1 or 3 ranks: the summed loss and
    the summed gradients agree (mass weights and the 1/trained-queries scale are normalised per unit)."""
    import torch
    corpus = A.synth_markov_corpus(1500, 12, 2, 8)
    trie = A.RadixTrie.build(corpus, 7, subtree_level=2)
    mf = MF.random_init(32, 2, 1, 12, 16, seed=3, std=0.2)
    counts = [torch.from_numpy(np.ascontiguousarray(c)).to(cuda) for c in (trie.cnt_off.astype(np.int32), trie.cnt_tok, trie.cnt_val)]
    results = []
    for world, rows in ((1, 100000), (1, 300), (3, 700)):
        total = None
        loss_sum, n_q = 0.0, 0
        for rank in range(world):
            groups, _ = T.build_groups(trie, rank, world, rows, "linear", mf.seq_len, cuda, level=2, unit_cap=120)
            model = T.TrieWalkModel(mf, cuda)
            for g in groups:
                ls, nq = model.group_step(g, counts, entropy_lambda=0.3)
                loss_sum += ls
                n_q += nq
            flat = model.flat_grad[:model.n_flat].double().cpu().numpy()
            total = flat if total is None else total + flat
        results.append((loss_sum, n_q, total))
    for loss_sum, n_q, total in results[1:]:
        assert n_q == results[0][1]
        assert abs(loss_sum - results[0][0]) / results[0][0] < 1e-5
        assert rel_err(total, results[0][2], floor=1e-6) < 1e-4


@pytest.mark.parametrize("sampler", [3, 4])
def test_lightning_unit_matches_dense_reference(cuda, sampler):
    """A sampled training unit (the sampled node's ancestors plus its subtree, or a root-to-leaf path; every row
    trained, as in the reference's executed code): loss and every weight gradient against the dense float64 model on
    the same rows."""
    import torch
    corpus = A.synth_markov_corpus(900, 12, 2, 13)
    trie = A.RadixTrie.build(corpus, 7)
    mf = MF.random_init(32, 2, 2, 12, 16, seed=6, std=0.2)
    counts_np = (trie.cnt_off.astype(np.int32), trie.cnt_tok, trie.cnt_val)
    counts = [torch.from_numpy(np.ascontiguousarray(c)).to(cuda) for c in counts_np]
    space = T.SampleSpace(trie)
    rs, na, off, _, nodes, _ = trie.lightning_sample(sampler, 4, 0x5c115e1, p_stop=0.4)
    checked = 0
    for s in range(4):
        ids = nodes[off[s]:off[s + 1]]
        g = space.group(ids, [], "linear", mf.seq_len, cuda)
        assert g.n == int(trie.edge_len[ids].sum()) and g.trained is None
        model = T.TrieWalkModel(mf, cuda)
        ls, nq = model.group_step(g, counts, entropy_lambda=0.2)
        tr = None if g.trained is None else g.trained.cpu().numpy()
        rl, rq, rg, _ = _reference(mf, g.plan.parent_dfs.copy(), g.tokens32.cpu().numpy(), g.plan.depth.copy(), g.q2n.cpu().numpy(),
                                   g.qoff.cpu().numpy(), g.rid.cpu().numpy(), counts_np,
                                   None if g.mass_w is None else g.mass_w.cpu().numpy(), 0.2, 1.0, tr, g.unit_of_row.cpu().numpy())
        assert nq == rq and abs(ls - rl) <= TOL_F32 * max(rl, 1e-6)
        # a root-to-leaf path is a handful of rows: bias gradients there are sums of a few terms that nearly cancel,
        # so float32 products leave 1e-4 of the largest entry; 3e-4 for these units
        for k, v in model.params.items():
            assert rel_err(v.grad.cpu().numpy().astype(np.float64), rg[k], floor=1e-6) < 3 * TOL_F32, k
        checked += nq
    assert checked > 0


def test_lightning_training_runs_from_the_command_line(cuda, tmp_path):
    corpus = A.synth_markov_corpus(3000, 20, 2, 5)
    trie = A.RadixTrie.build(corpus, 8)
    d = str(tmp_path / "trie")
    trie.save_dir(d, corpus.size, 20, A.token_hash(corpus))
    mf = MF.random_init(32, 2, 2, 20, 16, seed=2)
    mp, out = str(tmp_path / "m.model"), str(tmp_path / "out.model")
    MF.save(mp, mf)
    T.main(["--model", mp, "--trie-dir", d, "--epochs", "2", "--lr", "0.003", "--optimizer", "rmsprop", "--lightning-sampler", "l3",
            "--lightning-steps", "12", "--lightning-max-mass", "400", "--mass-weight", "log", "--lr-schedule", "warmup-cosine",
            "--warmup-epochs", "1", "--save", out])
    new = MF.load(out)
    assert all(np.isfinite(a).all() for _, a in new.mats)
    assert any(not np.array_equal(a, b) for (_, a), (_, b) in zip(mf.mats, new.mats))


@pytest.mark.parametrize("mode,keep", [("full", "all"), ("local_depth", "none"), ("own_edge", "own_edge")])
def test_trainer_step_matches_the_reference_model_restatement(cuda, mode, keep):
    """One step of the trainer against the CPU restatement of the reference's own per-node model step
    (oracle/model_oracle.py: src/agpt/incremental_forward.cr:14-217 + incremental_backward.cr:33-187 with the ancestor
    accumulators), for each of the reference's three dK/dV behaviours: persistent accumulators, accumulators dropped
    (src/agpt/trie_walk_trainer.cr:189) and own radix edge only (src/cuda/agpt_train.cu:5016-5020).  Loss and every
    weight gradient within the float32 parity tolerance."""
    import torch
    from tests.helpers import model_oracle_step
    corpus = A.synth_markov_corpus(420, 12, 2, 9)
    trie = A.RadixTrie.build(corpus, 7)
    mf = MF.random_init(32, 2, 2, 12, 16, seed=8, std=0.2)
    counts_np = (trie.cnt_off.astype(np.int32), trie.cnt_tok, trie.cnt_val)
    counts = [torch.from_numpy(np.ascontiguousarray(c)).to(cuda) for c in counts_np]
    groups, total = T.build_groups(trie, 0, 1, 10_000, "linear", mf.seq_len, cuda)
    assert len(groups) == 1
    g = groups[0]
    model = T.TrieWalkModel(mf, cuda)
    model.grad_mode = mode
    for p in model.parameters():
        p.grad = torch.zeros_like(p)
    ls, nq = model.group_step(g, counts, entropy_lambda=0.4, intermediate_weight=0.8)
    # the group's rows in its own depth-first order; the radix node of each row is its edge id
    rid = g.rid.cpu().numpy()
    edge_id = rid[g.q2n.cpu().numpy()]
    ol, oq, og, _ = model_oracle_step(mf, g.plan.parent_dfs.copy(), g.tokens32.cpu().numpy(), g.plan.depth.copy(), g.q2n.cpu().numpy(),
                                      g.qoff.cpu().numpy(), rid, counts_np, g.mass_w.cpu().numpy(), 0.4, 0.8, None,
                                      g.unit_of_row.cpu().numpy(), keep, edge_id)
    assert nq == oq and abs(ls - ol) <= TOL_F32 * ol
    for k, v in model.params.items():
        assert rel_err(v.grad.cpu().numpy().astype(np.float64), og[k], floor=1e-6) < TOL_F32, k
    if mode != "full":        # the truncated modes really differ from the full one in the K/V projections
        full = model_oracle_step(mf, g.plan.parent_dfs.copy(), g.tokens32.cpu().numpy(), g.plan.depth.copy(), g.q2n.cpu().numpy(),
                                 g.qoff.cpu().numpy(), rid, counts_np, g.mass_w.cpu().numpy(), 0.4, 0.8, None,
                                 g.unit_of_row.cpu().numpy())[2]
        assert rel_err(og["layer0.wk.w"], full["layer0.wk.w"], floor=1e-6) > 1e-2
