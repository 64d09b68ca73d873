"""Regenerates the golden vectors under tests/golden/ from the CPU oracle.

The reference cannot be run (no Crystal toolchain; its kernel dependency is not vendored), so
these are regression vectors of the oracle restatement, which is itself pinned by the reference's
spec constructions and trie-shape anchors (tests/test_oracle_pins.py).

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import agpt_b200 as A  # noqa: E402  (host-only calls: corpus generator)
from oracle import pyoracle as O  # noqa: E402


def main():
    corpus = A.synth_markov_corpus(600, 12, 2, 7)
    lv = O.Leveled(corpus, 6)
    rx = O.Radix(lv)
    parent, token, depth = rx.char_tree()
    n = parent.size
    H, hd = 2, 16
    rng = np.random.default_rng(1234)
    q, k, v, dout = [rng.standard_normal((n, H * hd)).astype(np.float32) for _ in range(4)]
    out, w, w_off, _ = O.attn_fwd(parent, H, hd, q, k, v)
    dq, dk, dv = O.attn_bwd(parent, H, hd, q, k, v, w, w_off, dout)
    np.savez_compressed(os.path.join(HERE, "attention_small.npz"), corpus=corpus, parent=parent, token=token,
                        depth=depth, H=H, hd=hd, q=q, k=k, v=v, dout=dout, out=out, dq=dq, dk=dk, dv=dv)
    # per-query loss over the whole trie as one chunk, radix nodes in id order
    R = rx.radix_count
    ids = np.arange(1, R, dtype=np.int32)
    el = rx.edge_len[ids]
    qoff = np.concatenate([[0], np.cumsum(el)]).astype(np.int32)
    q2n = np.repeat(np.arange(ids.size, dtype=np.int32), el)
    token_ids = np.concatenate([rx.edge_tok[rx.edge_off[r]:rx.edge_off[r + 1]] for r in ids]).astype(np.int32)
    V = 12
    logits = (rng.standard_normal((int(qoff[-1]), V)) * 1.5).astype(np.float32)
    mass_w = O.mass_weights(rx.edge_mass[ids], el, 3)
    lam, iw = 0.5, 0.7
    loss, grad = O.loss_per_query(logits, q2n, qoff, ids, token_ids, rx.cnt_off.astype(np.int32), rx.cnt_tok,
                                  rx.cnt_val, mass_w, lam, iw, False)
    np.savez_compressed(os.path.join(HERE, "loss_small.npz"), logits=logits, q2n=q2n, qoff=qoff, radix_ids=ids,
                        token_ids=token_ids, cnt_off=rx.cnt_off.astype(np.int32), cnt_tok=rx.cnt_tok,
                        cnt_val=rx.cnt_val, mass_w=mass_w, lam=lam, iw=iw, loss=loss, grad=grad,
                        edge_mass=rx.edge_mass[ids], edge_len=el)
    print("nodes", n, "queries", int(qoff[-1]), "radix", R - 1)


if __name__ == "__main__":
    main()
