"""CPU restatement of the reference's per-node model step for a whole (small) trie.  TEST INFRASTRUCTURE: only the
tests import it; the product never does.

Follows, function by function (paths inside the reference project):

* forward of one node            src/agpt/incremental_forward.cr:14-131  (embedding row, per block: LN1 -> x W + b for
                                 Q, K, V -> interleaved RoPE at position depth-1 -> attention over the node's
                                 root-to-node K/V rows -> WO + residual -> LN2 -> ReLU FFN + residual; final LN; logits)
* layer norm                     src/agpt/incremental_forward.cr:143-163 (float32, biased variance, eps 1e-5 inside the
                                 square root; the normalised row without gamma/beta is kept for the backward, :166-174)
* RoPE / inverse RoPE            src/agpt/incremental_forward.cr:201-225
* backward of one node           src/agpt/incremental_backward.cr:33-187 (output projection, final LN, blocks in reverse:
                                 FFN, LN2, WO, per-head attention backward with the descendants' accumulated dK/dV added
                                 at the node's own row, inverse RoPE on dQ and the node's dK, WQ/WK/WV, LN1, embedding row)
* layer-norm backward            src/agpt/incremental_backward.cr:212-243 (float64 means)
* softmax backward               src/agpt/incremental_backward.cr:245-253 (float64 dot)
* ancestor accumulators          src/agpt/node_state.cr:58-74, scatter src/agpt/trie_walk_trainer.cr:236-276; nodes are
                                 walked deepest first so that a node's accumulator is complete when the node is reached
                                 (persistent accumulators: the "full" gradient semantics).  keep = "none" drops the
                                 ancestor rows (src/agpt/trie_walk_trainer.cr:189), keep = "own_edge" keeps those on the
                                 node's own radix edge (src/cuda/agpt_train.cu:5016-5020).

Arithmetic is float32 with the float64 pieces named above; the row softmax is the usual max-shifted float32 one (the
reference calls its backend's softmax_rows, whose source is not in the reference project).
"""
from __future__ import annotations

import numpy as np

F = np.float32


def _ln_row(x, gamma, beta):
    d = x.size
    mean = F(x.sum(dtype=F) / F(d))
    diff = (x - mean).astype(F)
    var = F((diff * diff).sum(dtype=F) / F(d))
    std_inv = F(1.0 / np.sqrt(np.float64(F(var + F(1e-5)))))
    normed = (diff * std_inv).astype(F)
    return (normed * gamma + beta).astype(F), normed, std_inv


def _ln_backward_row(grad, normed, std_inv, gamma, dgamma, dbeta):
    dgamma += grad * normed
    dbeta += grad
    d_normed = (grad * gamma).astype(F)
    mean_dn = d_normed.astype(np.float64).mean()
    mean_dn_n = (d_normed.astype(np.float64) * normed.astype(np.float64)).mean()
    return ((d_normed.astype(np.float64) - mean_dn - normed.astype(np.float64) * mean_dn_n) * np.float64(std_inv)).astype(F)


def _rope(x, cos_row, sin_row, inverse=False):
    """x: [hd]; pairs (2i, 2i+1)."""
    out = x.copy()
    c, s = cos_row[0::2], sin_row[0::2]
    x0, x1 = x[0::2], x[1::2]
    if not inverse:
        out[0::2] = x0 * c - x1 * s
        out[1::2] = x0 * s + x1 * c
    else:
        out[0::2] = x0 * c + x1 * s
        out[1::2] = -x0 * s + x1 * c
    return out.astype(F)


def _softmax_row(s):
    e = np.exp((s - s.max()).astype(F)).astype(F)
    return (e / e.sum(dtype=F)).astype(F)


class ModelOracle:
    """params: dict name -> float32 array with the names of the MGPT matrix order (token_emb, layer{l}.wq.w, ...,
    final.gamma, out.w, out.b); cos, sin: RoPE tables [seq_len, head_dim]."""

    def __init__(self, params, d_model, n_heads, n_layers, cos, sin):
        self.P = {k: np.asarray(v, F) for k, v in params.items()}
        self.D, self.H, self.L = d_model, n_heads, n_layers
        self.hd = d_model // n_heads
        self.cos, self.sin = np.asarray(cos, F), np.asarray(sin, F)

    # ------------------------------------------------------------------------------------------------------------
    def forward(self, parent, tokens, positions):
        """Nodes in an order with parent[i] < i.  Returns logits [n, V]; keeps every node's state for backward()."""
        P, D, H, hd, L = self.P, self.D, self.H, self.hd, self.L
        n = parent.size
        self.parent, self.tokens, self.positions = parent, tokens, positions
        self.chain = []
        for i in range(n):
            self.chain.append((self.chain[parent[i]] if parent[i] >= 0 else []) + [i])
        self.K = np.zeros((L, n, D), F)
        self.V = np.zeros((L, n, D), F)
        self.state = [None] * n
        V_out = P["out.w"].shape[1]
        logits = np.zeros((n, V_out), F)
        scale = F(1.0 / np.sqrt(np.float64(hd)))
        for i in range(n):
            pos = int(positions[i])
            x = P["token_emb"][tokens[i]].copy()
            blocks = []
            for l in range(L):
                g = lambda name: P[f"layer{l}.{name}"]  # noqa: E731
                ln1_out, ln1_normed, ln1_si = _ln_row(x, g("ln1.gamma")[0], g("ln1.beta")[0])
                q = (ln1_out @ g("wq.w") + g("wq.b")[0]).astype(F)
                k = (ln1_out @ g("wk.w") + g("wk.b")[0]).astype(F)
                v = (ln1_out @ g("wv.w") + g("wv.b")[0]).astype(F)
                for h in range(H):
                    sl = slice(h * hd, (h + 1) * hd)
                    q[sl] = _rope(q[sl], self.cos[pos], self.sin[pos])
                    k[sl] = _rope(k[sl], self.cos[pos], self.sin[pos])
                self.K[l, i], self.V[l, i] = k, v
                ch = self.chain[i]
                weights, wo_in = [], np.zeros(D, F)
                for h in range(H):
                    sl = slice(h * hd, (h + 1) * hd)
                    sc = ((self.K[l, ch, sl] @ q[sl]).astype(F) * scale).astype(F)
                    w = _softmax_row(sc)
                    wo_in[sl] = (w @ self.V[l, ch, sl]).astype(F)
                    weights.append(w)
                x = (x + (wo_in @ g("wo.w") + g("wo.b")[0]).astype(F)).astype(F)
                ln2_out, ln2_normed, ln2_si = _ln_row(x, g("ln2.gamma")[0], g("ln2.beta")[0])
                hpre = (ln2_out @ g("l1.w") + g("l1.b")[0]).astype(F)
                mask = (hpre > 0).astype(F)
                relu_out = (hpre * mask).astype(F)
                x = (x + (relu_out @ g("l2.w") + g("l2.b")[0]).astype(F)).astype(F)
                blocks.append(dict(ln1_out=ln1_out, ln1_normed=ln1_normed, ln1_si=ln1_si, q=q, weights=weights, wo_in=wo_in,
                                   ln2_out=ln2_out, ln2_normed=ln2_normed, ln2_si=ln2_si, relu_out=relu_out, mask=mask))
            fin_out, fin_normed, fin_si = _ln_row(x, P["final.gamma"][0], P["final.beta"][0])
            logits[i] = (fin_out @ P["out.w"] + P["out.b"][0]).astype(F)
            self.state[i] = dict(blocks=blocks, fin_out=fin_out, fin_normed=fin_normed, fin_si=fin_si)
        return logits

    # ------------------------------------------------------------------------------------------------------------
    def backward(self, d_logits, keep="all", edge_id=None):
        """Weight gradients (dict like params) for the upstream gradient d_logits [n, V]; nodes deepest first."""
        P, D, H, hd, L = self.P, self.D, self.H, self.hd, self.L
        n = self.parent.size
        G = {k: np.zeros_like(v) for k, v in P.items()}
        acc_dk = np.zeros((L, n, D), F)
        acc_dv = np.zeros((L, n, D), F)
        scale = F(1.0 / np.sqrt(np.float64(hd)))
        for i in range(n - 1, -1, -1):
            st, pos, ch = self.state[i], int(self.positions[i]), self.chain[i]
            dl = np.asarray(d_logits[i], F)
            G["out.w"] += np.outer(st["fin_out"], dl)
            G["out.b"][0] += dl
            d_hidden = (dl @ P["out.w"].T).astype(F)
            d_hidden = _ln_backward_row(d_hidden, st["fin_normed"], st["fin_si"], P["final.gamma"][0], G["final.gamma"][0], G["final.beta"][0])
            for l in range(L - 1, -1, -1):
                g = lambda name: P[f"layer{l}.{name}"]  # noqa: E731
                gg = lambda name: G[f"layer{l}.{name}"]  # noqa: E731
                bs = st["blocks"][l]
                d_ff_out = d_hidden.copy()
                gg("l2.w")[...] += np.outer(bs["relu_out"], d_ff_out)
                gg("l2.b")[0] += d_ff_out
                d_relu = ((d_ff_out @ g("l2.w").T).astype(F) * bs["mask"]).astype(F)
                gg("l1.w")[...] += np.outer(bs["ln2_out"], d_relu)
                gg("l1.b")[0] += d_relu
                d_ln2_out = (d_relu @ g("l1.w").T).astype(F)
                d_hidden = (d_hidden + _ln_backward_row(d_ln2_out, bs["ln2_normed"], bs["ln2_si"], g("ln2.gamma")[0],
                                                        gg("ln2.gamma")[0], gg("ln2.beta")[0])).astype(F)
                d_attn_proj = d_hidden.copy()
                gg("wo.w")[...] += np.outer(bs["wo_in"], d_attn_proj)
                gg("wo.b")[0] += d_attn_proj
                d_concat = (d_attn_proj @ g("wo.w").T).astype(F)
                dq_all, dk_cur, dv_cur = np.zeros(D, F), np.zeros(D, F), np.zeros(D, F)
                for h in range(H):
                    sl = slice(h * hd, (h + 1) * hd)
                    w, d_out = bs["weights"][h], d_concat[sl]
                    k_h, v_h = self.K[l, ch, sl], self.V[l, ch, sl]
                    dv_full = np.outer(w, d_out).astype(F)
                    d_w = (v_h @ d_out).astype(F)
                    dot = float((d_w.astype(np.float64) * w.astype(np.float64)).sum())
                    d_sc = ((w.astype(np.float64) * (d_w.astype(np.float64) - dot)).astype(F) * scale).astype(F)
                    dq = (d_sc @ k_h).astype(F)
                    dk_full = np.outer(d_sc, bs["q"][sl]).astype(F)
                    dk_full[-1] += acc_dk[l, i, sl]
                    dv_full[-1] += acc_dv[l, i, sl]
                    for p_i, a in enumerate(ch[:-1]):
                        if keep == "all" or (keep == "own_edge" and edge_id[a] == edge_id[i]):
                            acc_dk[l, a, sl] += dk_full[p_i]
                            acc_dv[l, a, sl] += dv_full[p_i]
                    dq_all[sl] = _rope(dq, self.cos[pos], self.sin[pos], inverse=True)
                    dk_cur[sl] = _rope(dk_full[-1], self.cos[pos], self.sin[pos], inverse=True)
                    dv_cur[sl] = dv_full[-1]
                for name, grad in (("wq", dq_all), ("wk", dk_cur), ("wv", dv_cur)):
                    gg(f"{name}.w")[...] += np.outer(bs["ln1_out"], grad)
                    gg(f"{name}.b")[0] += grad
                d_ln1_out = ((dq_all @ g("wq.w").T).astype(F) + (dk_cur @ g("wk.w").T).astype(F) + (dv_cur @ g("wv.w").T).astype(F)).astype(F)
                d_hidden = (d_hidden + _ln_backward_row(d_ln1_out, bs["ln1_normed"], bs["ln1_si"], g("ln1.gamma")[0],
                                                        gg("ln1.gamma")[0], gg("ln1.beta")[0])).astype(F)
            G["token_emb"][self.tokens[i]] += d_hidden
        return G
