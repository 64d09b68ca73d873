"""Shared builders for the tests: random trees, the deterministic spec model, tolerances."""
from __future__ import annotations

import numpy as np

# Tolerances of the parity contract: float32 results within 1e-4 relative, bf16-store variants within
# 2e-2, both measured normwise (max |diff| over max |reference| of the tensor).
TOL_F32 = 1e-4
TOL_BF16 = 2e-2


def rel_err(a, b, floor=1e-2):
    """max |a - b| over max |b|; the denominator is floored so that a reference tensor that is exactly
    zero (a one-node tree has dq == 0) is compared absolutely at floor * tolerance."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    denom = max(np.abs(b).max(), floor)
    return float(np.abs(a - b).max() / denom)


def random_tree(n, max_depth, seed, branch_bias=0.5, roots=3):
    """Parent array with parent[i] < i (breadth-first-like ids), depth capped at max_depth."""
    rng = np.random.default_rng(seed)
    parent = np.full(n, -1, np.int32)
    depth = np.ones(n, np.int32)
    for i in range(roots, n):
        while True:
            lo = 0 if rng.random() < branch_bias else max(0, i - 8)
            p = int(rng.integers(lo, i))
            if depth[p] < max_depth:
                break
        parent[i] = p
        depth[i] = depth[p] + 1
    return parent


def chain_tree(n):
    return np.arange(-1, n - 1, dtype=np.int32)


def random_qkv(n, D, seed):
    rng = np.random.default_rng(seed)
    return [rng.standard_normal((n, D)).astype(np.float32) for _ in range(4)]


# ---- the deterministic model of the reference's backward-attention spec --------------------------------
def fill_mat(rows, cols, scale, offset=0):
    r = np.arange(rows)[:, None]
    c = np.arange(cols)[None, :]
    return ((((offset + r * cols + c) % 37) + 1).astype(np.float32) * np.float32(scale)).astype(np.float32)


class SpecModel:
    """d_model 8, heads [4, 4], one layer, d_ff 16, vocab 8, seq 8; weights from the fill rule
    value = ((offset + r*cols + c) % 37 + 1) * scale (spec/agpt_backward_attention_spec.cr:3-51)."""

    d_model, n_heads, hd, vocab, seq_len = 8, 2, 4, 8, 8

    def __init__(self):
        d = self.d_model
        self.token_emb = fill_mat(self.vocab, d, 0.01, 1)
        self.ln1_gamma = fill_mat(1, d, 0.02, 2)[0]
        self.ln1_beta = fill_mat(1, d, 0.01, 3)[0]
        self.wq_w, self.wq_b = fill_mat(d, d, 0.01, 6), fill_mat(1, d, 0.01, 7)[0]
        self.wk_w, self.wk_b = fill_mat(d, d, 0.01, 8), fill_mat(1, d, 0.01, 9)[0]
        self.wv_w, self.wv_b = fill_mat(d, d, 0.01, 10), fill_mat(1, d, 0.01, 11)[0]
        self.wo_w, self.wo_b = fill_mat(d, d, 0.01, 12), fill_mat(1, d, 0.01, 13)[0]

    def ln1(self, x):
        """float32 layer norm, biased variance, eps 1e-5 (src/agpt/incremental_forward.cr:143-163)."""
        x = x.astype(np.float32)
        mean = np.float32(0)
        for v in x:
            mean = np.float32(mean + v)
        mean = np.float32(mean / np.float32(x.size))
        var = np.float32(0)
        for v in x:
            diff = np.float32(v - mean)
            var = np.float32(var + diff * diff)
        var = np.float32(var / np.float32(x.size))
        sinv = np.float32(1.0 / np.sqrt(np.float64(np.float32(var + np.float32(1e-5)))))
        return ((x - mean) * sinv * self.ln1_gamma + self.ln1_beta).astype(np.float32)

    def qkv(self, token):
        """Pre-RoPE q, k, v rows and the LN1 output for one token (layer 0 input = embedding)."""
        xn = self.ln1(self.token_emb[token])
        q = (xn @ self.wq_w + self.wq_b).astype(np.float32)
        k = (xn @ self.wk_w + self.wk_b).astype(np.float32)
        v = (xn @ self.wv_w + self.wv_b).astype(np.float32)
        return q, k, v, xn


class MemTrie:
    """In-memory trie with insertion-order ids (src/agpt/trie_corpus.cr:200-228, :786-794, :897-913)."""

    def __init__(self, tokens, max_depth, max_starts=None, start_offset=0):
        self.parent, self.token, self.depth, self.children = [-1], [-1], [0], [dict()]
        self.counts = [dict()]
        n = len(tokens)
        total = n - 1
        if max_starts is None or max_starts >= total:
            starts = list(range(total))
        else:
            off = start_offset % total
            starts = [((i * total) // max_starts + off) % total for i in range(max_starts)]
        for s in starts:
            node, d, idx = 0, 0, s
            while idx < total and d < max_depth:
                tok, nxt = tokens[idx], tokens[idx + 1]
                ch = self.children[node].get(tok)
                if ch is None:
                    ch = len(self.parent)
                    self.parent.append(node); self.token.append(tok); self.depth.append(self.depth[node] + 1)
                    self.children.append(dict()); self.counts.append(dict())
                    self.children[node][tok] = ch
                node = ch
                self.counts[node][nxt] = self.counts[node].get(nxt, 0) + 1
                idx += 1
                d += 1

    def levels(self):
        """Breadth-first levels, children in token order (each_depth_level, :677-690)."""
        level, out = [0], []
        while level:
            out.append(level)
            nxt = []
            for v in level:
                nxt += [self.children[v][t] for t in sorted(self.children[v])]
            level = nxt
        return out


def suffix_order(corpus, key_len):
    """Start positions 0..n-2 ordered by their first key_len tokens (a shorter key orders before its extensions), and
    the number of equal leading tokens of neighbours: the input of the suffix-order trie builder, in plain Python."""
    c = [int(x) for x in corpus]
    n = len(c)
    sa = sorted(range(n - 1), key=lambda s: (tuple(c[s:s + key_len]), s))
    lcp = [0] * (n - 1)
    for i in range(1, n - 1):
        a, b = c[sa[i - 1]:sa[i - 1] + key_len], c[sa[i]:sa[i] + key_len]
        l = 0
        while l < len(a) and l < len(b) and a[l] == b[l]:
            l += 1
        lcp[i] = l
    return np.asarray(sa, np.int32), np.asarray(lcp, np.int32)


TRIE_ARRAYS = ("parent", "first_char_depth", "edge_len", "edge_mass", "endpoint_depth", "subtree_key", "edge_start", "edge_off",
               "edge_tok", "cnt_off", "cnt_tok", "cnt_val")


def assert_same_trie(a, b):
    assert (a.radix_count, a.n_depth_files, a.total_edge_chars, a.leveled_nodes) == \
        (b.radix_count, b.n_depth_files, b.total_edge_chars, b.leveled_nodes)
    for name in TRIE_ARRAYS:
        assert np.array_equal(getattr(a, name), getattr(b, name)), name


def suffix_order_np(corpus, key_len):
    """suffix_order() in numpy for corpora of millions of tokens: a lexicographic sort over key_len columns (a position
    past the end is column value -1), then the common leading tokens of neighbours column by column."""
    c = np.asarray(corpus, np.int64)
    n = c.size
    m = n - 1
    pad = np.concatenate([c, np.full(key_len, -1, np.int64)])
    starts = np.arange(m)
    sa = np.lexsort(tuple(pad[starts + d] for d in range(key_len - 1, -1, -1)) )     # last key is the primary one
    lcp = np.zeros(m, np.int64)
    alive = np.ones(m - 1, bool)
    a, b = sa[:-1], sa[1:]
    for d in range(key_len):
        same = alive & (pad[a + d] == pad[b + d]) & (pad[a + d] >= 0)
        lcp[1:] += same
        alive = same
    return sa.astype(np.int32), lcp.astype(np.int32)


def model_oracle_step(mf, parent, tokens, depth, q2n, qoff, rid, counts, mass_w, lam, iw, trained, unit_of_row, keep="all",
                      edge_id=None):
    """One launch group through the whole-model CPU oracle (oracle/model_oracle.py: the reference's per-node forward and
    backward) with the oracle's loss in between and the per-unit 1 / trained-queries scaling of the gradient rows.
    Returns (loss sum, trained queries, weight gradients, logits)."""
    from oracle import pyoracle as O
    from oracle.model_oracle import ModelOracle
    hd = mf.d_model // mf.n_heads
    cos, sin = O.rope_table(mf.seq_len, hd)
    mo = ModelOracle(dict(mf.mats), mf.d_model, mf.n_heads, mf.n_layers, cos, sin)
    pos = np.minimum(np.maximum(depth - 1, 0), mf.seq_len - 1)
    logits = mo.forward(np.asarray(parent), np.asarray(tokens), pos)
    loss, dlog = O.loss_per_query(logits, q2n, qoff, rid, tokens, *counts, mass_w, lam, iw)
    if trained is not None:
        loss = loss * trained
        dlog = dlog * trained[:, None]
    per_unit = np.bincount(unit_of_row, weights=(loss > 0).astype(np.float64), minlength=int(unit_of_row.max()) + 1)
    scale = np.where(per_unit > 0, 1.0 / np.maximum(per_unit, 1), 0.0)[unit_of_row]
    grads = mo.backward((dlog.astype(np.float64) * scale[:, None]).astype(np.float32), keep, edge_id)
    return float(loss[loss > 0].sum()), int((loss > 0).sum()), grads, logits
