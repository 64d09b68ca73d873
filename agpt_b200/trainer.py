"""Trie-walk trainer on top of the hot path: the walker, the per-subtree KV store and one epoch.

Mirrors the radix training loop of the reference trainer (src/cuda/agpt_train.cu:3177-5512): per launch
group (a forest of root-child or bigram subtrees in depth-first order) embed the edge characters, run every
layer (LN1, Q/K/V projections, RoPE, trie-scoped attention, WO, residual, LN2, ReLU FFN, residual), final LN and
output projection over all positions, per-query loss with mass weights normalised over the group, backward,
and an optimizer step.  The trie-scoped attention, its backward with ancestor dK/dV, RoPE and the loss are this
library's kernels; so are the dense projections (a tcgen05 float32-accurate GEMM), the layer norms, the bias / ReLU / column-sum
row kernels, the embedding gradient and the optimizer step; torch supplies the autograd tape, device memory and the
process group.  Model files (MGPT) and radix trie directories are read and written unchanged.

    python -m agpt_b200.trainer --model m.model --trie-dir DIR --epochs 3 --lr 3e-4 --optimizer rmsprop \\
        --rmsprop-beta 0.999 --mass-weight linear --save out.model
"""
from __future__ import annotations

import argparse
import os
import time

import numpy as np

from . import api as A
from . import model_file as MF


class LaunchGroup:
    """Rows of one launch: local forest (depth-first), tokens, RoPE positions and the loss index arrays.

    A launch packs several units (root-child or bigram subtrees).  What the reference normalises per chunk -- the
    mass weights by their mean (src/cuda/agpt_train.cu:4608-4637) and the gradient by the number of trained queries
    (:4834) -- is normalised here per unit (unit_of_row), so that results do not depend on how units are packed into
    launches or spread over ranks."""

    def __init__(self, parent, tokens, depth, radix_of, edge_mass, mass_mode, seq_len, device, tile=64, trained=None,
                 unit_of_row=None):
        import torch
        self.n = int(parent.size)
        self.plan = A.WalkerPlan(parent, tile, device.index if device.type == "cuda" else -1)   # a host-only plan on a CPU device (index arrays for tests)
        order = self.plan.dfs_to_node.astype(np.int64)
        assert np.array_equal(order, np.arange(self.n)), "launch groups are built in depth-first order"
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)  # noqa: E731
        self.tokens = t(tokens.astype(np.int64))
        self.tokens32 = t(tokens.astype(np.int32))
        self.pos = t(np.minimum(np.maximum(depth - 1, 0), seq_len - 1).astype(np.int32))
        starts = np.concatenate([[True], radix_of[1:] != radix_of[:-1]])
        if trained is not None:                      # a context row never shares a loss node with trained rows
            starts |= np.concatenate([[True], trained[1:] != trained[:-1]])
        unit_of_row = np.zeros(self.n, np.int64) if unit_of_row is None else np.asarray(unit_of_row, np.int64)
        starts |= np.concatenate([[True], unit_of_row[1:] != unit_of_row[:-1]])
        self.n_units = int(unit_of_row.max()) + 1 if self.n else 0
        self.unit_of_row = t(unit_of_row)
        # rows of a unit are consecutive in every group build_groups makes: per-unit sums are then differences of a
        # running sum at these offsets (no scattered adds)
        self.unit_off = None
        if self.n and np.all(unit_of_row[1:] >= unit_of_row[:-1]):
            self.unit_off = t(np.searchsorted(unit_of_row, np.arange(self.n_units + 1)).astype(np.int64))
        qoff = np.concatenate([np.nonzero(starts)[0], [self.n]]).astype(np.int32)
        rid = radix_of[starts].astype(np.int32)
        self.q2n = t((np.cumsum(starts) - 1).astype(np.int32))
        self.qoff = t(qoff)
        self.rid = t(rid)
        counted = np.ones(rid.size, bool) if trained is None else trained[starts]
        mw = (A.mass_weights_by_unit(edge_mass[rid], np.diff(qoff), unit_of_row[starts], counted, self.n_units, mass_mode)
              if mass_mode != "off" else None)
        self.edge_first = t(A.edge_first_positions(radix_of))    # for the own-edge gradient mode
        self.trained = None if trained is None else t(trained.astype(np.float32))
        self.mass_w = None if mw is None else t(mw)
        self.n_trained_rows = self.n if trained is None else int(trained.sum())


def build_groups(trie: A.RadixTrie, rank: int, world: int, group_rows: int, mass_mode: str, seq_len: int, device,
                 tile: int = 64, level: int | None = None, unit_cap: int | None = None):
    """This rank's launch groups: root-child units (one rank) or bigram units balanced over ranks, packed in
    depth-first order into groups of at most group_rows rows.  With unit_cap, units larger than that are cut deeper
    (WalkerPlan.units_capped), which bounds the activation memory of a launch.  A unit that does not start at depth 1
    carries its ancestors as context rows (attended, and differentiated through, but not trained), so every chain is
    complete and the summed gradient does not depend on the partition."""
    parent, token, depth, radix_of = trie.char_tree()
    gplan = A.WalkerPlan(parent, 64, -1)
    if level is None:
        level = 1 if world == 1 else 2
    ub, ue = gplan.units(level) if unit_cap is None else gplan.units_capped(level, unit_cap)
    owner = A.partition_lpt(ue - ub, world)
    d2n = gplan.dfs_to_node
    groups = []
    for par, row, tr, unit in A.launch_groups(gplan, ub, ue, owner, rank, group_rows):
        idv = d2n[row]
        groups.append(LaunchGroup(par, token[idv], depth[idv], radix_of[idv], trie.edge_mass, mass_mode, seq_len, device, tile,
                                  None if tr.all() else tr, unit))
    return groups, int(gplan.n)


def _embedding_function():
    import torch

    class TokenEmbedding(torch.autograd.Function):
        """Row gather; the gradient of the table is summed per symbol in a fixed order (with a vocabulary of tens of
        symbols and millions of rows an index_put backward serialises on the collisions)."""

        @staticmethod
        def forward(ctx, emb, tokens32):
            ctx.save_for_backward(tokens32)
            ctx.vocab = emb.shape[0]
            return A.embedding_gather(emb, tokens32)

        @staticmethod
        def backward(ctx, grad):
            (tokens32,) = ctx.saved_tensors
            return A.embedding_grad(grad.contiguous(), tokens32, ctx.vocab), None

    return TokenEmbedding


def _layer_norm_function():
    import torch

    class RowLayerNorm(torch.autograd.Function):
        """Layer norm over the last dimension with the library's kernels (saved state: normalised rows, 1/std)."""

        @staticmethod
        def forward(ctx, x, gamma, beta):
            y, norm, sinv = A.layer_norm_forward(x.contiguous(), gamma.contiguous(), beta.contiguous())
            ctx.save_for_backward(norm, sinv, gamma)
            return y

        @staticmethod
        def backward(ctx, grad):
            norm, sinv, gamma = ctx.saved_tensors
            dgamma, dbeta = torch.zeros_like(gamma), torch.zeros_like(gamma)
            dx = A.layer_norm_backward(grad.contiguous(), norm, sinv, gamma.contiguous(), dgamma, dbeta)
            return dx, dgamma, dbeta

    return RowLayerNorm


def _norm_skip_function():
    import torch

    class NormWithSkip(torch.autograd.Function):
        """Layer norm of the residual stream x, returned together with x for the skip connection.  The two gradients
        that come back -- through the normalised rows and through the skip -- are added inside the layer-norm
        backward kernel instead of in a pass of their own (the reference's launch_elem_add after each
        cuda_layer_norm_backward, src/cuda/agpt_train.cu:4907-4909, :5066-5068)."""

        @staticmethod
        def forward(ctx, x, gamma, beta):
            x = x.contiguous()
            y, norm, sinv = A.layer_norm_forward(x, gamma.contiguous(), beta.contiguous())
            ctx.save_for_backward(norm, sinv, gamma)
            return y, x.view_as(x)

        @staticmethod
        def backward(ctx, grad, grad_skip):
            norm, sinv, gamma = ctx.saved_tensors
            dgamma, dbeta = torch.zeros_like(gamma), torch.zeros_like(gamma)
            add = None if grad_skip is None else grad_skip.contiguous()
            if grad is None:
                return add, dgamma, dbeta
            dx = A.layer_norm_backward(grad.contiguous(), norm, sinv, gamma.contiguous(), dgamma, dbeta, add=add)
            return dx, dgamma, dbeta

    return NormWithSkip


def _weight_grad(x, grad, w):
    """x^T grad with the row dimension cut into slices that are summed in a fixed order."""
    tiles = -(-w.shape[0] // 128) * -(-w.shape[1] // 128)
    split_k = max(1, min(x.shape[0] // 2048, -(-296 // tiles)))
    return A.gemm_f32(x, grad, trans_a=True, split_k=split_k)


def _qkv_function():
    import torch

    class QKVProjection(torch.autograd.Function):
        """q, k, v = x W + b for the three projections that read the same normalised rows
        (src/cuda/agpt_train.cu:4675-4683).  Backward (:5026-5061): the three input gradients are accumulated by the GEMMs
        themselves (the second and third take the running sum as their source matrix and write it back in place)."""

        @staticmethod
        def forward(ctx, x, wq, bq, wk, bk, wv, bv):
            x = x.contiguous()
            ctx.save_for_backward(x, wq, wk, wv)
            return A.gemm_f32(x, wq, bias=bq), A.gemm_f32(x, wk, bias=bk), A.gemm_f32(x, wv, bias=bv)

        @staticmethod
        def backward(ctx, dq, dk, dv):
            x, wq, wk, wv = ctx.saved_tensors
            dx, out = None, []
            for g, w in ((dq, wq), (dk, wk), (dv, wv)):
                g = g.contiguous()
                db, _ = A.col_sum(g)
                dx = A.gemm_f32(g, w, trans_b=True, residual=dx, out=dx)
                out += [_weight_grad(x, g, w), db]
            return (dx, *out)

    return QKVProjection


def _linear_function():
    import torch

    class TensorLinear(torch.autograd.Function):
        """y = x @ w + b (+ residual; relu: max(., 0)) in one GEMM launch of the library.  Backward: the
        ReLU mask and the bias gradient are one pass over the incoming gradient; the weight gradient cuts the row
        dimension into slices that are summed in a fixed order."""

        @staticmethod
        def forward(ctx, x, w, b, relu, residual):
            x = x.contiguous()
            y = A.gemm_f32(x, w, bias=b, relu=relu, residual=None if residual is None else residual.contiguous())
            ctx.relu, ctx.has_residual = relu, residual is not None
            ctx.save_for_backward(x, w, y if relu else None)
            return y

        @staticmethod
        def backward(ctx, grad):
            x, w, y = ctx.saved_tensors
            grad = grad.contiguous()
            if ctx.relu:
                db, grad = A.col_sum(grad, act=y, grad_out=torch.empty_like(grad))
            else:
                db, _ = A.col_sum(grad)
            dx = A.gemm_f32(grad, w, trans_b=True)
            return dx, _weight_grad(x, grad, w), db, None, (grad if ctx.has_residual else None)

    return TensorLinear


def _attention_function():
    import torch

    class TrieAttention(torch.autograd.Function):
        """RoPE + trie-scoped attention; backward returns gradients w.r.t. the pre-RoPE q and k."""

        @staticmethod
        def forward(ctx, q, k, v, group, cos, sin, n_heads, bf16_store, grad_mode="full"):
            # q and k are rotated in place: they are fresh projection outputs that nothing else reads or saves
            q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
            A.rope_pair_(q, k, group.pos, cos, sin, n_heads)
            ks, vs = (A.kv_store_write_bf16(k), A.kv_store_write_bf16(v)) if bf16_store else (k, v)
            out, lse = A.attn_forward(group.plan, q, ks, vs, n_heads)
            ctx.save_for_backward(q, ks, vs, out, lse)
            ctx.group, ctx.cos, ctx.sin, ctx.n_heads, ctx.grad_mode = group, cos, sin, n_heads, grad_mode
            return out

        @staticmethod
        def backward(ctx, dout):
            q, ks, vs, out, lse = ctx.saved_tensors
            dq, dk, dv = A.attn_backward(ctx.group.plan, q, ks, vs, out, lse, dout.contiguous(), ctx.n_heads,
                                         grad_mode=ctx.grad_mode, edge_first=ctx.group.edge_first)
            A.rope_pair_(dq, dk, ctx.group.pos, ctx.cos, ctx.sin, ctx.n_heads, inverse=True)
            return dq, dk, dv, None, None, None, None, None, None

    return TrieAttention


class TrieWalkModel:
    """Parameters of an MGPT model as torch tensors on one device, and the per-group forward/backward."""

    def __init__(self, model: MF.Model, device):
        import torch
        self.cfg = model
        self.device = device
        # one flat weight buffer and one flat gradient buffer (the reference's d_weights / d_grads), each matrix on a
        # 16-byte boundary; the gradient buffer ends with the epoch's loss sum and query count (three floats) so that
        # one all-reduce carries everything
        offs, off = [], 0
        for _, a in model.mats:
            offs.append(off)
            off += (a.size + 3) & ~3
        self.n_flat = off
        self.flat = torch.zeros(off, dtype=torch.float32, device=device)
        self.flat_grad = torch.zeros(off + 4, dtype=torch.float32, device=device)
        self.params = {}
        for (name, a), o in zip(model.mats, offs):
            p = self.flat[o:o + a.size].view(a.shape)
            p.copy_(torch.from_numpy(np.ascontiguousarray(a)))
            self.params[name] = p.requires_grad_(True)
        self._offs = offs
        self.bind_grads()
        hd = model.d_model // model.n_heads
        cos, sin = A.rope_table(model.seq_len, hd)
        self.cos, self.sin = torch.from_numpy(cos).to(device), torch.from_numpy(sin).to(device)
        self.attn = _attention_function()
        self.embed = _embedding_function()
        self.ln = _layer_norm_function()
        self.linear = _linear_function()
        self.norm_skip = _norm_skip_function()
        self.qkv = _qkv_function()
        self.dense_impl = "tensor"       # "tensor": the library's 3xTF32 GEMM; "torch": torch.addmm (cuBLAS float32)
        self.ffn_recompute = False       # True: recompute the d_ff-wide activations in the backward instead of keeping them
        # which attention pairs feed dK/dV: "full" (persistent accumulators, src/agpt/incremental_backward.cr), "local_depth"
        # (the Crystal walker, src/agpt/trie_walk_trainer.cr:189) or "own_edge" (the CUDA trainer, src/cuda/agpt_train.cu:5016-5020)
        self.grad_mode = "full"

    def parameters(self):
        return list(self.params.values())

    def bind_grads(self):
        """Make every parameter's .grad the matching slice of the flat gradient buffer (autograd accumulates in place)."""
        for p, o in zip(self.params.values(), self._offs):
            want = self.flat_grad[o:o + p.numel()].view(p.shape)
            if p.grad is None or p.grad.data_ptr() != want.data_ptr():
                p.grad = want

    def to_model_file(self) -> MF.Model:
        m = self.cfg
        out = MF.Model(m.d_model, m.n_heads, m.n_layers, m.d_ff, m.vocab, m.seq_len)
        out.mats = [(name, self.params[name].detach().cpu().numpy().copy()) for name, _ in m.mats]
        return out

    def logits(self, group: LaunchGroup, bf16_store=False):
        import torch
        from torch.utils.checkpoint import checkpoint
        P, m = self.params, self.cfg
        ln = self.ln.apply

        def lin(x, w, b, relu=False, residual=None):
            # the library GEMM needs 16-byte aligned rows; other widths (a vocabulary of 65) go to torch
            if self.dense_impl == "tensor" and w.shape[0] % 4 == 0 and w.shape[1] % 4 == 0:
                return self.linear.apply(x, w, b, relu, residual)
            y = torch.addmm(b, x, w)
            y = torch.relu(y) if relu else y
            return y if residual is None else residual + y

        def ffn(x, g2, b2, w1, b1, w2, bo):
            return lin(lin(ln(x, g2, b2), w1, b1, relu=True), w2, bo, residual=x)

        fused = self.dense_impl == "tensor" and m.d_model % 4 == 0 and m.d_ff % 4 == 0
        x = self.embed.apply(P["token_emb"], group.tokens32)
        for l in range(m.n_layers):
            g = lambda n: P[f"layer{l}.{n}"]  # noqa: E731
            if fused:
                x1, skip = self.norm_skip.apply(x, g("ln1.gamma")[0], g("ln1.beta")[0])
                q, k, v = self.qkv.apply(x1, g("wq.w"), g("wq.b")[0], g("wk.w"), g("wk.b")[0], g("wv.w"), g("wv.b")[0])
            else:
                x1, skip = ln(x, g("ln1.gamma")[0], g("ln1.beta")[0]), x
                q = lin(x1, g("wq.w"), g("wq.b")[0])
                k = lin(x1, g("wk.w"), g("wk.b")[0])
                v = lin(x1, g("wv.w"), g("wv.b")[0])
            a = self.attn.apply(q, k, v, group, self.cos, self.sin, m.n_heads, bf16_store, self.grad_mode)
            x = lin(a, g("wo.w"), g("wo.b")[0], residual=skip)
            args = (x, g("ln2.gamma")[0], g("ln2.beta")[0], g("l1.w"), g("l1.b")[0], g("l2.w"), g("l2.b")[0])
            if self.ffn_recompute:
                x = checkpoint(ffn, *args, use_reentrant=False)
            elif fused:
                x2, skip = self.norm_skip.apply(x, args[1], args[2])
                x = lin(lin(x2, args[3], args[4], relu=True), args[5], args[6], residual=skip)
            else:
                x = ffn(*args)
        xf = ln(x, P["final.gamma"][0], P["final.beta"][0])
        w, b = P["out.w"], P["out.b"][0]
        pad = (-m.vocab) % 4
        if pad and self.dense_impl == "tensor":
            # A vocabulary that is not a multiple of 4 (65 symbols) would leave rows off a 16-byte boundary, which the
            # library GEMM does not take.  The projection is padded to the next multiple of 4: zero weight columns and a
            # bias of -1e30 there, so the extra logits have probability exactly 0, contribute nothing to any loss and
            # receive a zero gradient; the padding is differentiable (its backward is a slice), so out.w and out.b get
            # their gradients as before.
            w = torch.nn.functional.pad(w, (0, pad))
            b = torch.cat([b, torch.full((pad,), -1e30, dtype=b.dtype, device=b.device)])
        return lin(xf, w, b)

    def group_step(self, group: LaunchGroup, counts, entropy_lambda=0.0, intermediate_weight=1.0, ce_only=False,
                   bf16_store=False, sync=True):
        """Forward, loss and backward of one launch group; gradients accumulate into .grad.
        Returns (sum of positive per-query losses, number of such queries): Python numbers, or with sync=False a
        float32 device tensor (loss sum, count // 4096, count % 4096), so that the host does not wait for the device
        between groups."""
        import torch
        logits = self.logits(group, bf16_store).contiguous()
        c_off, c_tok, c_val = counts
        if logits.shape[1] != self.cfg.vocab:
            # padded vocabulary: the entropy weight 1 + lambda H / ln V (src/cuda/agpt_train.cu:2147-2160) is taken with the
            # true V, so lambda is rescaled by ln(padded V) / ln(V) for the kernel, which divides by ln of the row width
            entropy_lambda = entropy_lambda * float(np.log(logits.shape[1]) / np.log(self.cfg.vocab))
        loss, dlogits = A.loss_per_query(logits.detach(), group.q2n, group.qoff, group.rid, group.tokens32, c_off, c_tok,
                                         c_val, group.mass_w, entropy_lambda, intermediate_weight, ce_only)
        if group.trained is not None:               # context rows carry no loss
            loss = loss * group.trained
            dlogits = dlogits * group.trained[:, None]
        pos = loss > 0
        n_trained = pos.sum()
        loss_sum = torch.where(pos, loss, torch.zeros_like(loss)).sum(dtype=torch.float64)
        # every gradient row is scaled by 1 / (trained queries of its unit): the reference's per-chunk scaling
        # (src/cuda/agpt_train.cu:4834) with the unit as the chunk
        if group.unit_off is not None:
            run = torch.nn.functional.pad(torch.cumsum(pos, 0, dtype=torch.int32), (1, 0))
            per_unit = (run[group.unit_off[1:]] - run[group.unit_off[:-1]]).to(torch.float32)
        else:
            per_unit = torch.zeros(group.n_units, dtype=torch.float32, device=loss.device).index_add_(0, group.unit_of_row, pos.to(torch.float32))
        scale = torch.where(per_unit > 0, 1.0 / per_unit.clamp(min=1.0), torch.zeros_like(per_unit))
        logits.backward(dlogits * scale[group.unit_of_row][:, None])
        if sync:
            return float(loss_sum.item()), int(n_trained.item())
        # the count rides in float32 next to the gradients: split so that sums over groups and ranks stay exact
        return torch.stack([loss_sum.to(torch.float32), (n_trained // 4096).to(torch.float32), (n_trained % 4096).to(torch.float32)])


class SampleSpace:
    """What building the launch group of a sampled node set needs: the char tree of the whole trie in depth-first order."""

    def __init__(self, trie: A.RadixTrie):
        self.trie = trie
        self.parent, self.token, self.depth, self.radix_of = trie.char_tree()
        self.plan = A.WalkerPlan(self.parent, 64, -1)

    def group(self, node_ids, context_ids, mass_mode, seq_len, device, tile=64) -> LaunchGroup:
        """Launch group of the chars of the radix nodes node_ids (closed under "parent"); chars of context_ids are
        attended but carry no loss and are left out of the mass-weight mean.  The lightning samplers pass no context:
        in the reference the ancestors prepended to a sampled subtree are trained like every other position and counted
        in the chunk's mass mean (src/cuda/agpt_train.cu:4601-4637; the ancestor count recorded at :4194 is never read,
        and the comment at :4160-4180 that announces a masking describes a variant that was taken out again)."""
        t = self.trie
        node_ids = np.asarray(node_ids, np.int64)
        lens = t.edge_len[node_ids].astype(np.int64)
        starts = t.edge_start[node_ids].astype(np.int64)
        chars = np.repeat(starts - np.concatenate([[0], np.cumsum(lens)[:-1]]), lens) + np.arange(int(lens.sum()))
        pos = self.plan.node_to_dfs[chars].astype(np.int64)
        order = np.argsort(pos, kind="stable")
        chars, pos = chars[order], pos[order]
        ppos = self.plan.parent_dfs[pos].astype(np.int64)
        local_parent = np.where(ppos < 0, -1, np.searchsorted(pos, ppos)).astype(np.int32)
        if np.any((ppos >= 0) & (pos[np.minimum(local_parent, pos.size - 1)] != ppos)):
            raise ValueError("the node set is not closed under parent")
        trained = ~np.isin(self.radix_of[chars], np.asarray(context_ids, np.int64))
        return LaunchGroup(local_parent, self.token[chars], self.depth[chars], self.radix_of[chars], t.edge_mass, mass_mode, seq_len,
                           device, tile, None if trained.all() else trained)


def lightning_lr_weights(masses, mode: str) -> np.ndarray:
    """Per-sample learning-rate multipliers of the reference's --mass-lr (src/cuda/agpt_train.cu:4276-4300): the summed
    edge mass of each sample compressed (log(1+m), sqrt(m) or m) and divided by the mean over the super-epoch's samples."""
    m = np.asarray(masses, np.float64)
    if mode == "off" or m.size == 0:
        return np.ones(m.size, np.float64)
    c = np.log(1.0 + m) if mode == "log" else (np.where(m > 0, np.sqrt(np.maximum(m, 0.0)), 0.0) if mode == "sqrt" else m.copy())
    total = float(c.sum())
    mean = total / m.size if total > 0.0 else 1.0
    return c / mean


def train_lightning_epoch(model: TrieWalkModel, space: SampleSpace, counts, opt, sampler: int, steps: int, rng_state: int,
                          mass_mode="off", p_stop=0.3, max_mass=0, mass_lr="off", **loss_kw):
    """One super-epoch of the reference's lightning mode: `steps` sampled units, each its own gradient and optimizer step
    (src/cuda/agpt_train.cu:152-157).  Returns (loss sum, queries, nodes trained, new generator state)."""
    rs, na, off, masses, nodes, rng_state = space.trie.lightning_sample(sampler, steps, rng_state, p_stop, max_mass)
    lr_w = lightning_lr_weights(masses, mass_lr)
    model.bind_grads()
    loss_sum, n_q, n_nodes = 0.0, 0, 0
    for s in range(steps):
        ids = nodes[off[s]:off[s + 1]]
        # every sampled row is trained, the ancestors the sampler prepends included (src/cuda/agpt_train.cu:4601-4607)
        g = space.group(ids, [], mass_mode, model.cfg.seq_len, model.device)
        opt.zero_grad(set_to_none=False)
        ls, nq = model.group_step(g, counts, **loss_kw)
        if hasattr(opt, "lr_scale"):
            opt.lr_scale = float(lr_w[s])
        opt.step()
        loss_sum += ls
        n_q += nq
        n_nodes += int(ids.size)
    return loss_sum, n_q, n_nodes, rng_state


class FlatOptimizer:
    """The library's fused step (clip, update, decay, clear gradients) over the model's flat buffers."""

    def __init__(self, model, kind, lr, beta1, beta2, eps, weight_decay=0.0, clip_norm=0.0):
        import torch
        self.model, self.kind, self.lr, self.beta1, self.beta2, self.eps = model, kind, lr, beta1, beta2, eps
        self.base_lr = lr
        self.weight_decay, self.clip_norm, self.t = weight_decay, clip_norm, 0
        self.schedule = None             # (name, total steps, warm-up steps): lr of each step from A.compute_lr
        self.lr_scale = 1.0              # per-step multiplier (the lightning mode's learning rate by sample mass)
        z = lambda: torch.zeros(model.n_flat, dtype=torch.float32, device=model.device)  # noqa: E731
        self.m = z() if kind in ("momentum", "adam") else None
        self.v = z() if kind in ("rmsprop", "adam") else None

    def step(self):
        if self.schedule is not None:
            name, total, warm = self.schedule
            self.lr = A.compute_lr(self.base_lr, self.t, total, warm, name)
        self.t += 1
        m = self.model
        return A.optimizer_step(self.kind, m.flat, m.flat_grad[:m.n_flat], self.m, self.v, lr=self.lr * self.lr_scale, beta1=self.beta1,
                                beta2=self.beta2, eps=self.eps, t=self.t, weight_decay=self.weight_decay,
                                clip_norm=self.clip_norm, zero_grads=True)

    def zero_grad(self, set_to_none=False):
        self.model.flat_grad.zero_()


def make_optimizer(name, model, lr, rmsprop_beta=0.999, adam_betas=(0.9, 0.999), momentum=0.9, eps=1e-8, weight_decay=0.0,
                   clip_norm=0.0):
    """Optimizer over a TrieWalkModel (the library's fused step) or, given a plain parameter list, torch's own."""
    import torch
    if isinstance(model, TrieWalkModel):
        beta1 = momentum if name == "momentum" else adam_betas[0]
        beta2 = rmsprop_beta if name == "rmsprop" else adam_betas[1]
        if name not in A.OPTIMIZER_KINDS:
            raise ValueError(f"unknown optimizer {name}")
        return FlatOptimizer(model, name, lr, beta1, beta2, eps, weight_decay, clip_norm)
    params = model
    if name == "sgd":
        return torch.optim.SGD(params, lr=lr)
    if name == "momentum":
        return torch.optim.SGD(params, lr=lr, momentum=momentum)
    if name == "rmsprop":
        return torch.optim.RMSprop(params, lr=lr, alpha=rmsprop_beta, eps=eps)
    if name == "adam":
        return torch.optim.Adam(params, lr=lr, betas=adam_betas, eps=eps)
    raise ValueError(f"unknown optimizer {name}")


def train_epoch(model: TrieWalkModel, groups, counts, opt, accumulate=True, world=1, **loss_kw):
    """One sweep over every position of this rank's groups.  accumulate=True: gradients of all groups (and all
    ranks) are summed and one optimizer step closes the epoch; False: one step per group (single rank only).
    The loss sum and query count ride at the end of the flat gradient buffer: one all-reduce, one host read."""
    import torch.distributed as dist
    model.bind_grads()
    opt.zero_grad(set_to_none=False)
    tail = model.flat_grad[model.n_flat:model.n_flat + 3]
    for g in groups:
        tail += model.group_step(g, counts, sync=False, **loss_kw)
        if not accumulate:
            opt.step()                       # clears the parameter gradients, not the two statistics behind them
    if accumulate:
        if world > 1:
            dist.all_reduce(model.flat_grad)
        opt.step()
    stats = tail.cpu()
    return float(stats[0]), int(round(float(stats[1]))) * 4096 + int(round(float(stats[2])))


def main(argv=None):
    import torch
    import torch.distributed as dist
    ap = argparse.ArgumentParser(description="trie-walk training on a radix trie directory")
    ap.add_argument("--model", required=True)
    ap.add_argument("--trie-dir", required=True)
    ap.add_argument("--save", default=None)
    ap.add_argument("--save-every", type=int, default=0)
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--optimizer", default="adam", choices=["sgd", "momentum", "rmsprop", "adam"])
    ap.add_argument("--rmsprop-beta", type=float, default=0.999)
    ap.add_argument("--lr-schedule", default="constant", choices=["constant", "cosine", "warmup-cosine"])
    ap.add_argument("--warmup-epochs", type=int, default=0)
    ap.add_argument("--weight-decay", type=float, default=0.0)
    ap.add_argument("--grad-clip-norm", type=float, default=0.0)
    ap.add_argument("--mass-weight", default="off", choices=["off", "log", "sqrt", "linear"])
    ap.add_argument("--entropy-lambda", type=float, default=0.0)
    ap.add_argument("--intermediate-weight", type=float, default=1.0)
    ap.add_argument("--ce-only", action="store_true")
    ap.add_argument("--no-accumulate", action="store_true")
    ap.add_argument("--bf16-kv", action="store_true")
    ap.add_argument("--grad-mode", default="full", choices=["full", "local_depth", "own_edge"],
                    help="attention pairs that feed dK/dV: every descendant (default), the node's own query, or the queries on the key's radix edge")
    ap.add_argument("--group-rows", type=int, default=1_000_000)
    ap.add_argument("--ffn-recompute", action="store_true", help="recompute the FFN activations in the backward (less memory)")
    ap.add_argument("--lightning-sampler", default=None, choices=["l1", "l2", "l3", "l4"],
                    help="stochastic training units instead of the deterministic sweep (one rank)")
    ap.add_argument("--lightning-steps", type=int, default=65)
    ap.add_argument("--lightning-p-stop", type=float, default=0.3)
    ap.add_argument("--lightning-seed", type=lambda v: int(v, 0), default=0x5c115e1)
    ap.add_argument("--lightning-max-mass", type=int, default=0)
    ap.add_argument("--lightning-mass-lr", default="off", choices=["off", "log", "sqrt", "linear"])
    ap.add_argument("--partition-depth", type=int, default=0, choices=[0, 1, 2],
                    help="1 = root-child units, 2 = bigram units; 0 = 1 on one rank, 2 on several")
    args = ap.parse_args(argv)

    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    if not torch.cuda.is_available():
        raise SystemExit("agpt_b200.trainer needs a CUDA device")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    mf = MF.load(args.model)
    trie = A.RadixTrie.load_dir(args.trie_dir)
    if rank == 0:
        print(f"  Model: d={mf.d_model} heads={mf.n_heads} layers={mf.n_layers} ff={mf.d_ff} vocab={mf.vocab} seq={mf.seq_len}")
        print(f"  Radix trie: {trie.radix_count} nodes, {trie.total_edge_chars} total edge chars, {trie.n_depth_files} endpoint depths")
    lightning = args.lightning_sampler is not None
    if lightning and world > 1:
        raise SystemExit("lightning sampling runs on one rank")
    if lightning:
        space, groups, total = SampleSpace(trie), [], trie.total_edge_chars
    else:
        groups, total = build_groups(trie, rank, world, args.group_rows, args.mass_weight, mf.seq_len, dev,
                                     level=args.partition_depth or None)
    rng_state = args.lightning_seed
    counts = [torch.from_numpy(np.ascontiguousarray(c)).to(dev) for c in (trie.cnt_off.astype(np.int32), trie.cnt_tok, trie.cnt_val)]
    model = TrieWalkModel(mf, dev)
    model.ffn_recompute = args.ffn_recompute
    model.grad_mode = args.grad_mode
    opt = make_optimizer(args.optimizer, model, args.lr, args.rmsprop_beta, weight_decay=args.weight_decay,
                         clip_norm=args.grad_clip_norm)
    n_sub = int((trie.parent[1:] == 0).sum())
    # optimizer steps per epoch, as the reference counts them for its schedule (src/cuda/agpt_train.cu:5100-5117)
    per_epoch = args.lightning_steps if lightning else (len(groups) if (args.no_accumulate and world == 1) else 1)
    if args.lr_schedule != "constant":
        opt.schedule = (args.lr_schedule, max(per_epoch * args.epochs, 1), args.warmup_epochs * per_epoch)
    save = args.save or args.model
    for ep in range(1, args.epochs + 1):
        torch.cuda.synchronize()
        t0 = time.time()
        loss_kw = dict(entropy_lambda=args.entropy_lambda, intermediate_weight=args.intermediate_weight, ce_only=args.ce_only,
                       bf16_store=args.bf16_kv)
        if lightning:
            ls, nq, _, rng_state = train_lightning_epoch(model, space, counts, opt, int(args.lightning_sampler[1]), args.lightning_steps,
                                                         rng_state, args.mass_weight, args.lightning_p_stop, args.lightning_max_mass,
                                                         mass_lr=args.lightning_mass_lr, **loss_kw)
            units, chunks = args.lightning_steps, args.lightning_steps
        else:
            ls, nq = train_epoch(model, groups, counts, opt, accumulate=not args.no_accumulate or world > 1, world=world, **loss_kw)
            units, chunks = n_sub, len(groups)
        torch.cuda.synchronize()
        if rank == 0:
            print(f"Epoch {ep}: loss={ls / max(nq, 1):.6f}  ({time.time() - t0:.2f} sec, {units} subtrees, {chunks} chunks, {nq} nodes)",
                  flush=True)
            if args.save_every and ep % args.save_every == 0:
                MF.save(f"{save}.ep{ep}", model.to_model_file())
    if rank == 0:
        MF.save(save, model.to_model_file())
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
