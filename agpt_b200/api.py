"""Host-side mirror of the reference's operator interface for the trie-walk hot path.

Everything here forwards to the C ABI in ``libagpt_b200.so``; torch supplies device
memory and streams only.  Names follow the reference: a *trie* (radix, with edges), its
*char positions*, a *walker plan* over the char tree, the per-subtree *KV store*, and the
legacy ``cuda_batched_varlen_attention*`` kernels.
"""
from __future__ import annotations

import ctypes as C
import math
import os

import numpy as np

from ._lib import AgptError, GroupInfo, PlanInfo, TrieInfo, check, lib

KV_F32, KV_BF16 = 0, 1


def _np_i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _vp(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _view(ptr, n, dtype):
    """Copy of a C array owned by a library handle (the copy outlives the handle)."""
    if n == 0:
        return np.zeros(0, dtype=dtype)
    return np.ctypeslib.as_array(ptr, shape=(int(n),)).astype(dtype, copy=True)


# ----------------------------------------------------------------------------------------
# synthetic workloads
# ----------------------------------------------------------------------------------------
def synth_markov_corpus(n: int, vocab: int, order: int, seed: int = 0, repeat_log2: int = 0) -> np.ndarray:
    """Seeded order-`order` Markov corpus with Zipf(1.1) marginals; repeat_log2 > 0 injects, with probability
    2^-repeat_log2 per position, a copy of 64..256 symbols from an earlier offset (long verbatim repeats)."""
    out = np.zeros(n, np.int32)
    if repeat_log2:
        check(lib().agpt_b200_synth_markov_corpus_repeats(n, vocab, order, seed, repeat_log2, _vp(out)), "synth_markov_corpus_repeats")
    else:
        check(lib().agpt_b200_synth_markov_corpus(n, vocab, order, seed, _vp(out)), "synth_markov_corpus")
    return out


def synth_tree(max_nodes: int, max_depth: int = 64, root_children: int = 65, p_stop: float = 0.35,
               max_children: int = 65, level_cap: int = 75_000, seed: int = 0) -> np.ndarray:
    """Parent array (breadth-first ids, -1 under the root) of the attention microbenchmark tree."""
    out = np.zeros(max_nodes, np.int32)
    n = check(lib().agpt_b200_synth_tree(max_nodes, max_depth, root_children, p_stop, max_children, level_cap,
                                         seed, _vp(out)), "synth_tree")
    return out[:n].copy()


# ----------------------------------------------------------------------------------------
# radix trie
# ----------------------------------------------------------------------------------------
class RadixTrie:
    """Radix trie with the reference's node numbering, counts, edge mass and char positions."""

    def __init__(self, handle):
        self._h = handle
        info = TrieInfo()
        check(lib().agpt_b200_trie_info(handle, C.byref(info)), "trie_info")
        R = info.radix_count
        self.radix_count, self.n_depth_files = R, info.n_depth_files
        self.total_edge_chars = int(info.total_edge_chars)
        self.leveled_nodes = int(info.leveled_nodes)
        for name in ("parent", "first_char_depth", "edge_len", "edge_mass", "endpoint_depth", "subtree_key",
                     "edge_start"):
            setattr(self, name, _view(getattr(info, name), R, np.int32))
        self.edge_off = _view(info.edge_off, R + 1, np.int64)
        self.edge_tok = _view(info.edge_tok, self.total_edge_chars, np.int32)
        self.cnt_off = _view(info.cnt_off, R + 1, np.int64)
        self.cnt_tok = _view(info.cnt_tok, info.total_counts, np.int32)
        self.cnt_val = _view(info.cnt_val, info.total_counts, np.int32)

    @classmethod
    def build(cls, corpus, max_depth: int, subtree_level: int = 1, prune_min_mass: int = 1,
              prune_min_depth: int = 4) -> "RadixTrie":
        c = _np_i32(corpus)
        h = C.c_void_p()
        check(lib().agpt_b200_trie_build(_vp(c), c.size, max_depth, subtree_level, prune_min_mass, prune_min_depth,
                                         C.byref(h)), "trie_build")
        return cls(h)

    @classmethod
    def build_gpu(cls, corpus, max_depth: int, subtree_level: int = 1, prune_min_mass: int = 1, prune_min_depth: int = 4,
                  device: int = 0) -> "RadixTrie":
        """The same trie as build(), with the suffix ordering done on the GPU.  A corpus shorter than max_depth + 2
        tokens (nothing to order) goes to the level-by-level builder."""
        c = _np_i32(corpus)
        if c.size < max_depth + 2:
            return cls.build(c, max_depth, subtree_level, prune_min_mass, prune_min_depth)
        h = C.c_void_p()
        check(lib().agpt_b200_trie_build_gpu(_vp(c), c.size, max_depth, subtree_level, prune_min_mass, prune_min_depth, device,
                                             C.byref(h)), "trie_build_gpu")
        return cls(h)

    @classmethod
    def from_suffix_order(cls, corpus, max_depth: int, sa, lcp, subtree_level: int = 1, prune_min_mass: int = 1,
                          prune_min_depth: int = 4) -> "RadixTrie":
        """The same trie as build(), assembled from a given suffix order (see agpt_b200_trie_from_suffix_order)."""
        c, sa, lcp = _np_i32(corpus), _np_i32(sa), _np_i32(lcp)
        h = C.c_void_p()
        check(lib().agpt_b200_trie_from_suffix_order(_vp(c), c.size, max_depth, subtree_level, prune_min_mass, prune_min_depth,
                                                     _vp(sa), _vp(lcp), C.byref(h)), "trie_from_suffix_order")
        return cls(h)

    @classmethod
    def load_dir(cls, path: str) -> "RadixTrie":
        h = C.c_void_p()
        check(lib().agpt_b200_trie_load_dir(path.encode(), C.byref(h)), "trie_load_dir")
        return cls(h)

    @classmethod
    def load_subtree(cls, path: str, key: int) -> "RadixTrie":
        """One per-subtree file of a radix directory as a trie of its own (local ids, 0 = root)."""
        h = C.c_void_p()
        check(lib().agpt_b200_trie_load_subtree(path.encode(), int(key), C.byref(h)), "trie_load_subtree")
        return cls(h)

    @staticmethod
    def manifest(path: str):
        """(keys, radix nodes, edge chars, deepest endpoint) of the per-subtree files listed in manifest.bin."""
        n = check(lib().agpt_b200_trie_manifest(path.encode(), 0, None, None, None, None), "trie_manifest")
        keys, nodes, ep = np.zeros(n, np.int32), np.zeros(n, np.int32), np.zeros(n, np.int32)
        chars = np.zeros(n, np.int64)
        check(lib().agpt_b200_trie_manifest(path.encode(), n, _vp(keys), _vp(nodes), _vp(chars), _vp(ep)), "trie_manifest")
        return keys, nodes, chars, ep

    def save_dir(self, path: str, corpus_tokens: int, vocab: int, corpus_hash: int,
                 tag: str = "char.sorted_unique.v1", per_subtree: bool = False):
        os.makedirs(path, exist_ok=True)
        if per_subtree:
            os.makedirs(os.path.join(path, "subtrees"), exist_ok=True)
        check(lib().agpt_b200_trie_save_dir(self._h, path.encode(), int(per_subtree), corpus_tokens, vocab,
                                            corpus_hash, tag.encode()), "trie_save_dir")

    def lightning_sample(self, sampler: int, steps: int, rng_state: int, p_stop: float = 0.3, max_mass: int = 0):
        """`steps` stochastic training units (see agpt_b200_lightning_sample).  Returns (sampled radix ids, ancestor
        counts, node offsets, masses, node ids, new generator state)."""
        st = C.c_uint32(rng_state)
        total = lib().agpt_b200_lightning_sample(self._h, sampler, steps, p_stop, max_mass, C.byref(st), None, None, None, None, None, 0)
        if total < 0:
            check(int(total), "lightning_sample")
        rs, na = np.zeros(steps, np.int32), np.zeros(steps, np.int32)
        off, mass, nodes = np.zeros(steps + 1, np.int64), np.zeros(steps, np.float64), np.zeros(max(int(total), 1), np.int32)
        got = lib().agpt_b200_lightning_sample(self._h, sampler, steps, p_stop, max_mass, C.byref(st), _vp(rs), _vp(na), _vp(off),
                                               _vp(mass), _vp(nodes), nodes.size)
        if got < 0:
            check(int(got), "lightning_sample")
        return rs, na, off, mass, nodes[:int(total)], int(st.value)

    def char_tree(self):
        """(parent, token, depth, radix_of_char) per char position, trainer numbering."""
        n = self.total_edge_chars
        out = [np.zeros(n, np.int32) for _ in range(4)]
        check(lib().agpt_b200_trie_char_tree(self._h, *[_vp(a) for a in out]), "trie_char_tree")
        return tuple(out)

    def close(self):
        if self._h is not None:
            lib().agpt_b200_trie_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def token_hash(tokens) -> int:
    t = _np_i32(tokens)
    return int(lib().agpt_b200_token_hash(_vp(t), t.size))


# ----------------------------------------------------------------------------------------
# walker plan
# ----------------------------------------------------------------------------------------
class WalkerPlan:
    """Depth-first layout of a tree plus the tile index the attention kernels walk."""

    def __init__(self, parent, tile_m: int = 64, device: int = -1):
        par = _np_i32(parent)
        h = C.c_void_p()
        check(lib().agpt_b200_plan_create(_vp(par), par.size, tile_m, device, C.byref(h)), "plan_create")
        self._h = h
        info = PlanInfo()
        check(lib().agpt_b200_plan_info(h, C.byref(info)), "plan_info")
        self.info = info
        n = int(info.n)
        self.n, self.tile_m, self.n_tiles = n, info.tile_m, int(info.n_tiles)
        self.max_depth, self.sum_depth = info.max_depth, int(info.sum_depth)
        self.sum_group_prefix, self.n_groups = int(info.sum_group_prefix), int(info.n_groups)
        self.chain_rows = int(info.chain_rows)
        # kernels one backward launches: the tile kernel plus the reduction passes that have work
        self.bwd_launches = 1 + int(info.n_reduce_items > 0) + int(info.n_reduce_multi > 0)
        self.dfs_to_node = _view(info.dfs_to_node, n, np.int32)
        self.node_to_dfs = _view(info.node_to_dfs, n, np.int32)
        self.parent_dfs = _view(info.parent_dfs, n, np.int32)
        self.depth = _view(info.depth, n, np.int32)
        self.sub_end = _view(info.sub_end, n, np.int32)
        self.device = info.device

    def workspace_bytes(self, d_model: int) -> int:
        return check(lib().agpt_b200_attn_bwd_workspace_bytes(self._h, d_model), "attn_bwd_workspace_bytes")

    def units(self, level: int = 1):
        """Root-child (level 1) or bigram (level 2) units as depth-first [begin, end) ranges."""
        cnt = check(lib().agpt_b200_plan_units(self._h, level, 0, None, None), "plan_units")
        b = np.zeros(cnt, np.int64)
        e = np.zeros(cnt, np.int64)
        check(lib().agpt_b200_plan_units(self._h, level, cnt, _vp(b), _vp(e)), "plan_units")
        return b, e

    def units_capped(self, level: int, cap: int):
        """Units of at most `cap` rows where the tree allows it: a unit larger than cap is cut into the unary chain
        at its top (up to and including the first branching node) and the subtrees below it, recursively -- the
        reference's partition by deeper ancestor groups (--partition-depth, src/cuda/agpt_train.cu:3808-3890), applied
        only where a subtree is too large.  Depth-first [begin, end) ranges in depth-first order; a range is a whole
        subtree or such a chain."""
        ub, ue = self.units(level)
        sub_end = self.sub_end
        out_b, out_e = [], []
        stack = [(int(b), int(e)) for b, e in zip(ub[::-1], ue[::-1])]
        while stack:
            b, e = stack.pop()
            if e - b <= cap:
                out_b.append(b)
                out_e.append(e)
                continue
            j = b
            while j + 1 < e and int(sub_end[j + 1]) == e:        # exactly one child: the chain goes on
                j += 1
            if j + 1 >= e:                                        # a bare chain: nothing to cut
                out_b.append(b)
                out_e.append(e)
                continue
            out_b.append(b)
            out_e.append(j + 1)
            kids, c = [], j + 1
            while c < e:
                kids.append((c, int(sub_end[c])))
                c = int(sub_end[c])
            stack.extend(reversed(kids))
        return np.asarray(out_b, np.int64), np.asarray(out_e, np.int64)

    def algorithmic_bytes(self, d_model: int, n_heads: int, kv_bytes: int = 4):
        """Bytes of the sibling-group-shared traffic model for one forward+backward of one layer:
        each sibling group reads its parent's ancestor chain once per direction and every per-node
        tensor is read or written once."""
        D, H, b, N = d_model, n_heads, kv_bytes, self.n
        fwd = self.sum_group_prefix * 2 * D * b + N * (D * 4 + 2 * D * b + D * 4 + H * 4)
        bwd = self.sum_group_prefix * 2 * D * b + N * (3 * D * 4 + 2 * H * 4 + 2 * D * b + D * 4 + 2 * D * 4)
        return fwd, bwd

    def close(self):
        if self._h is not None:
            lib().agpt_b200_plan_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def launch_groups(plan: WalkerPlan, unit_begin, unit_end, unit_rank, rank: int, group_rows: int):
    """This rank's units packed into launch groups (agpt_b200_groups_create).  Returns a list of
    (local parent int32, plan position of each row int64, trained bool, unit_of_row int32)."""
    ub = np.ascontiguousarray(unit_begin, dtype=np.int64)
    ue = np.ascontiguousarray(unit_end, dtype=np.int64)
    ur = None if unit_rank is None else _np_i32(unit_rank)
    h = C.c_void_p()
    check(lib().agpt_b200_groups_create(plan._h, _vp(ub), _vp(ue), None if ur is None else _vp(ur), ub.size, rank, int(group_rows),
                                        C.byref(h)), "groups_create")
    out = []
    try:
        for i in range(int(lib().agpt_b200_groups_count(h))):
            info = GroupInfo()
            check(lib().agpt_b200_groups_get(h, i, C.byref(info)), "groups_get")
            n = int(info.n)
            out.append((_view(info.parent, n, np.int32).copy(), _view(info.row, n, np.int64).copy(),
                        _view(info.trained, n, np.uint8).astype(bool), _view(info.unit_of_row, n, np.int32).copy()))
    finally:
        lib().agpt_b200_groups_free(h)
    return out


def partition_lpt(unit_weight, n_ranks: int) -> np.ndarray:
    w = np.ascontiguousarray(unit_weight, dtype=np.int64)
    out = np.zeros(w.size, np.int32)
    check(lib().agpt_b200_partition_lpt(_vp(w), w.size, n_ranks, _vp(out)), "partition_lpt")
    return out


def shard_tree(parent, rank: int, n_ranks: int, level: int = 2):
    """Nodes of `rank`'s share of a tree partitioned by root-child (level 1) or bigram (level 2)
    subtree, longest-processing-time balanced on unit size.  Returns (local_parent, node_ids,
    is_context): the sub-forest's parent array, the original ids of its nodes, and a mask of
    context-only rows (a depth-1 ancestor kept so its descendants' chains stay complete while the
    node itself is trained by another rank)."""
    parent = _np_i32(parent)
    plan = WalkerPlan(parent, 64, -1)
    ub, ue = plan.units(level)
    owner = partition_lpt(ue - ub, n_ranks)
    mine = np.zeros(plan.n, bool)
    for b, e, o in zip(ub, ue, owner):
        if o == rank:
            mine[b:e] = True
    ctx = np.zeros(plan.n, bool)
    if level == 2:
        # depth-1 ancestors of owned depth>=2 rows ride along as context
        pos = np.nonzero(mine)[0]
        if pos.size:
            d1 = pos.copy()
            # walk up to depth 1 using subtree intervals: depth-1 ancestor = last depth-1 start <= pos
            starts = np.nonzero(plan.depth == 1)[0]
            d1 = starts[np.searchsorted(starts, pos, side="right") - 1]
            need = np.unique(d1)
            ctx[need[~mine[need]]] = True
    keep = mine | ctx
    pos = np.nonzero(keep)[0]
    remap = np.full(plan.n, -1, np.int64)
    remap[pos] = np.arange(pos.size)
    pp = plan.parent_dfs[pos]
    local_parent = np.where(pp < 0, -1, remap[np.maximum(pp, 0)]).astype(np.int32)
    node_ids = plan.dfs_to_node[pos].copy()
    return local_parent, node_ids, ctx[pos].copy()


# ----------------------------------------------------------------------------------------
# device entry points (torch tensors on the plan's device)
# ----------------------------------------------------------------------------------------
def _stream():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dp(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _chk_f32(t, name):
    import torch
    if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous():
        raise AgptError(f"{name} must be a contiguous float32 CUDA tensor")


def gather_rows(src, index):
    import torch
    _chk_f32(src, "src")
    out = torch.empty((index.numel(), src.shape[1]), dtype=torch.float32, device=src.device)
    check(lib().agpt_b200_gather_rows(_dp(src), _dp(index), _dp(out), index.numel(), src.shape[1], _stream()),
          "gather_rows")
    return out


def rope_table(max_seq: int, head_dim: int, base: float = 10000.0):
    """cos/sin tables [max_seq, head_dim], float32 host arithmetic, pair-duplicated."""
    c = np.zeros((max_seq, head_dim), np.float32)
    s = np.zeros((max_seq, head_dim), np.float32)
    check(lib().agpt_b200_rope_table(_vp(c), _vp(s), max_seq, head_dim, base), "rope_table")
    return c, s


def rope_(x, pos, cos, sin, n_heads: int, inverse: bool = False):
    """Rotate x [n, n_heads*head_dim] in place by per-row positions."""
    _chk_f32(x, "x")
    hd = x.shape[1] // n_heads
    check(lib().agpt_b200_rope(_dp(x), _dp(pos), _dp(cos), _dp(sin), x.shape[0], n_heads, hd, int(inverse), _stream()),
          "rope")
    return x


def rope_pair_(a, b, pos, cos, sin, n_heads: int, inverse: bool = False):
    """rope_ of two matrices of one shape (q and k, or their gradients) in one launch."""
    _chk_f32(a, "a")
    _chk_f32(b, "b")
    if a.shape != b.shape:
        raise AgptError("rope_pair_: the two matrices differ in shape")
    hd = a.shape[1] // n_heads
    check(lib().agpt_b200_rope_pair(_dp(a), _dp(b), _dp(pos), _dp(cos), _dp(sin), a.shape[0], n_heads, hd, int(inverse), _stream()),
          "rope_pair")
    return a, b


_gemm_ws = {}


def gemm_f32(a, b, trans_a=False, trans_b=False, bias=None, out=None, split_k=1, residual=None, relu=False):
    """out = act(op(a) @ op(b) + residual + bias row), float32 on the tensor cores with float32-level accuracy.
    a, b (and residual): contiguous 2-D float32 CUDA tensors."""
    import torch
    _chk_f32(a, "a")
    _chk_f32(b, "b")
    M, K = (a.shape[1], a.shape[0]) if trans_a else a.shape
    K2, N = (b.shape[1], b.shape[0]) if trans_b else b.shape
    if K != K2:
        raise AgptError(f"gemm_f32: inner dimensions differ ({K} vs {K2})")
    out = torch.empty((M, N), dtype=torch.float32, device=a.device) if out is None else out
    need = lib().agpt_b200_gemm_f32_workspace_bytes(int(trans_a), int(trans_b), M, N, K, split_k)
    if need < 0:
        check(int(need), "gemm_f32_workspace_bytes")
    ws = _gemm_ws.get(a.device.index)
    if need and (ws is None or ws.numel() < need):
        ws = _gemm_ws[a.device.index] = torch.empty(int(need), dtype=torch.uint8, device=a.device)
    if residual is not None:
        _chk_f32(residual, "residual")
        if tuple(residual.shape) != (M, N):
            raise AgptError("gemm_f32: residual shape differs from the output's")
    check(lib().agpt_b200_gemm_f32(int(trans_a), int(trans_b), M, N, K, 1.0, _dp(a), a.shape[1], _dp(b), b.shape[1],
                                   1.0 if residual is not None else 0.0, _dp(residual), N, _dp(bias), int(relu), _dp(out), N, split_k,
                                   _dp(ws) if need else None, int(need), _stream()), "gemm_f32")
    return out


def layer_norm_forward(x, gamma, beta):
    """y = norm * gamma + beta; returns (y, norm, std_inv) with the reference's saved state."""
    import torch
    _chk_f32(x, "x")
    rows, cols = x.shape
    y, norm = torch.empty_like(x), torch.empty_like(x)
    sinv = torch.empty(rows, dtype=torch.float32, device=x.device)
    check(lib().agpt_b200_layer_norm_fwd(_dp(x), _dp(y), _dp(norm), _dp(sinv), _dp(gamma), _dp(beta), rows, cols, _stream()),
          "layer_norm_fwd")
    return y, norm, sinv


def layer_norm_backward(grad, norm, sinv, gamma, dgamma, dbeta, add=None):
    """dx (returned); dgamma and dbeta are accumulated into.  add [rows, cols]: a gradient added to dx in the same
    pass (what reaches the same rows by the residual path)."""
    import torch
    _chk_f32(grad, "grad")
    rows, cols = grad.shape
    if add is not None:
        _chk_f32(add, "add")
        if tuple(add.shape) != (rows, cols):
            raise AgptError("layer_norm_backward: add has another shape than grad")
    dx = torch.empty_like(grad)
    wsb = check(lib().agpt_b200_layer_norm_bwd_workspace_bytes(rows, cols), "layer_norm_bwd_workspace_bytes")
    ws = torch.empty(wsb, dtype=torch.uint8, device=grad.device)
    check(lib().agpt_b200_layer_norm_bwd_add(_dp(grad), _dp(norm), _dp(sinv), _dp(gamma), _dp(add), _dp(dx), _dp(dgamma), _dp(dbeta),
                                             rows, cols, _dp(ws), wsb, _stream()), "layer_norm_bwd")
    return dx


def kv_store_write_bf16(src):
    import torch
    _chk_f32(src, "src")
    out = torch.empty(src.shape, dtype=torch.bfloat16, device=src.device)
    check(lib().agpt_b200_kv_store_write_bf16(_dp(src), _dp(out), src.shape[0], src.shape[1], _stream()),
          "kv_store_write_bf16")
    return out


def _kv_dtype(k):
    import torch
    if k.dtype == torch.float32:
        return KV_F32
    if k.dtype == torch.bfloat16:
        return KV_BF16
    raise AgptError("KV store must be float32 or bfloat16")


def validate_attn_args(plan: WalkerPlan, n_heads: int, f32_rows=(), kv_rows=(), lse=None, require_cuda: bool = True):
    """Refuse, before anything is launched, tensors the attention entry points would read or write out of bounds:
    the C entry points take no row count (it is the plan's), so a tensor with fewer rows than the plan, another
    width, dtype, device or a non-contiguous layout must be caught here.  f32_rows / kv_rows: (name, tensor) pairs
    that must be [plan.n, D] float32, resp. float32 or bfloat16; lse: [plan.n, n_heads] float32.  Returns (D, hd)."""
    import torch
    if not f32_rows:
        raise AgptError("no tensors given")
    ref = f32_rows[0][1]
    if ref.dim() != 2:
        raise AgptError(f"{f32_rows[0][0]} must be 2-D [rows, n_heads * head_dim]")
    D = int(ref.shape[1])
    if n_heads < 1 or D % n_heads:
        raise AgptError(f"width {D} is not a multiple of n_heads {n_heads}")
    hd = D // n_heads
    if hd not in (16, 32, 64):
        raise AgptError(f"head_dim {hd} unsupported (16, 32 or 64)")

    def one(name, t, dtypes, shape):
        if tuple(t.shape) != shape:
            raise AgptError(f"{name} has shape {tuple(t.shape)}, the plan needs {shape}")
        if t.dtype not in dtypes:
            raise AgptError(f"{name} has dtype {t.dtype}, expected one of {[str(d) for d in dtypes]}")
        if not t.is_contiguous():
            raise AgptError(f"{name} must be contiguous")
        if require_cuda and not t.is_cuda:
            raise AgptError(f"{name} must be a CUDA tensor")
        if t.device != ref.device:
            raise AgptError(f"{name} is on {t.device}, {f32_rows[0][0]} on {ref.device}")
        if require_cuda and plan.device >= 0 and t.device.index != plan.device:
            raise AgptError(f"{name} is on {t.device}, the plan on cuda:{plan.device}")

    for name, t in f32_rows:
        one(name, t, (torch.float32,), (plan.n, D))
    for name, t in kv_rows:
        one(name, t, (torch.float32, torch.bfloat16), (plan.n, D))
    if len(kv_rows) == 2 and kv_rows[0][1].dtype != kv_rows[1][1].dtype:
        raise AgptError("k and v must have the same dtype")
    if lse is not None:
        one("lse", lse, (torch.float32,), (plan.n, n_heads))
    return D, hd


def attn_forward(plan: WalkerPlan, q, k, v, n_heads: int, scale: float | None = None, out=None, lse=None):
    import torch
    _chk_f32(q, "q")
    n, D = q.shape
    hd = D // n_heads
    out = torch.empty_like(q) if out is None else out
    lse = torch.empty((n, n_heads), dtype=torch.float32, device=q.device) if lse is None else lse
    validate_attn_args(plan, n_heads, [("q", q), ("out", out)], [("k", k), ("v", v)], lse)
    scale = 1.0 / math.sqrt(hd) if scale is None else scale
    check(lib().agpt_b200_attn_fwd(plan._h, _dp(q), _dp(k), _dp(v), _kv_dtype(k), _dp(out), _dp(lse), n_heads, hd,
                                   scale, _stream()), "attn_fwd")
    return out, lse


GRAD_MODES = {"full": 0, "local_depth": 1, "own_edge": 2}


def edge_first_positions(edge_id) -> np.ndarray:
    """For rows in depth-first order with their radix node id: the row index of the first char of each row's edge
    (the chars of one edge are consecutive rows)."""
    e = np.asarray(edge_id)
    starts = np.concatenate([[True], e[1:] != e[:-1]])
    return np.maximum.accumulate(np.where(starts, np.arange(e.size), 0)).astype(np.int32)


def attn_backward(plan: WalkerPlan, q, k, v, out, lse, dout, n_heads: int, scale: float | None = None,
                  workspace=None, dq=None, dk=None, dv=None, grad_mode: str = "full", edge_first=None):
    """grad_mode: which attention pairs feed dK/dV -- "full" (a node and all its descendants), "local_depth" (the
    node's own query only) or "own_edge" (the queries on the key's own radix edge; edge_first: int32 tensor [n], see
    edge_first_positions).  dQ is the same in all three."""
    import torch
    _chk_f32(q, "q")
    _chk_f32(dout, "dout")
    n, D = q.shape
    hd = D // n_heads
    scale = 1.0 / math.sqrt(hd) if scale is None else scale
    if workspace is None:
        workspace = torch.empty(plan.workspace_bytes(D), dtype=torch.uint8, device=q.device)
    dq = torch.empty_like(q) if dq is None else dq
    dk = torch.empty_like(q) if dk is None else dk
    dv = torch.empty_like(q) if dv is None else dv
    validate_attn_args(plan, n_heads, [("q", q), ("out", out), ("dout", dout), ("dq", dq), ("dk", dk), ("dv", dv)],
                       [("k", k), ("v", v)], lse)
    if workspace.dtype != torch.uint8 or not workspace.is_contiguous() or workspace.device != q.device:
        raise AgptError("workspace must be a contiguous uint8 tensor on the device of q")
    if grad_mode not in GRAD_MODES:
        raise AgptError(f"grad_mode {grad_mode!r}: one of {sorted(GRAD_MODES)}")
    if grad_mode == "own_edge":
        if edge_first is None or edge_first.dtype != torch.int32 or tuple(edge_first.shape) != (plan.n,) or \
                not edge_first.is_contiguous() or edge_first.device != q.device:
            raise AgptError("own_edge needs edge_first: a contiguous int32 tensor [plan.n] on the device of q")
    check(lib().agpt_b200_attn_bwd_mode(plan._h, _dp(q), _dp(k), _dp(v), _kv_dtype(k), _dp(out), _dp(lse), _dp(dout),
                                        _dp(dq), _dp(dk), _dp(dv), _dp(workspace), workspace.numel(), n_heads, hd, scale,
                                        GRAD_MODES[grad_mode], _dp(edge_first) if grad_mode == "own_edge" else None,
                                        _stream()), "attn_bwd")
    return dq, dk, dv


_scratch = {}


def _workspace(device, key, nbytes):
    """A per-device scratch tensor kept between calls (grown on demand)."""
    import torch
    t = _scratch.get((device.index, key))
    if t is None or t.numel() < nbytes:
        t = _scratch[(device.index, key)] = torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=device)
    return t


def bias_act(x, bias, relu=False, out=None, mask=None):
    """out = x + bias, or max(x + bias, 0) with an optional 0/1 mask; out may be x itself."""
    import torch
    _chk_f32(x, "x")
    _chk_f32(bias, "bias")
    out = torch.empty_like(x) if out is None else out
    check(lib().agpt_b200_bias_act(_dp(x), _dp(bias), _dp(out), _dp(mask), x.shape[0], x.shape[1], int(relu), _stream()), "bias_act")
    return out


def relu_backward(grad, mask, out=None):
    import torch
    _chk_f32(grad, "grad")
    _chk_f32(mask, "mask")
    out = torch.empty_like(grad) if out is None else out
    check(lib().agpt_b200_relu_bwd(_dp(grad), _dp(mask), _dp(out), grad.numel(), _stream()), "relu_bwd")
    return out


def col_sum(grad, act=None, grad_out=None, out=None, scale=1.0, accumulate=False):
    """Column sums of grad [rows, cols] (a bias gradient).  With act, grad is first masked by act > 0 and the
    masked gradient is written to grad_out (default: in place).  Returns (sums, masked gradient or None)."""
    import torch
    _chk_f32(grad, "grad")
    rows, cols = grad.shape
    if act is not None:
        _chk_f32(act, "act")
        grad_out = grad if grad_out is None else grad_out
    out = torch.zeros(cols, dtype=torch.float32, device=grad.device) if out is None else out
    wsb = check(lib().agpt_b200_col_sum_workspace_bytes(rows, cols), "col_sum_workspace_bytes")
    ws = _workspace(grad.device, "col_sum", wsb)
    check(lib().agpt_b200_col_sum(_dp(grad), _dp(act), _dp(grad_out), rows, cols, scale, int(accumulate), _dp(out), _dp(ws), wsb,
                                  _stream()), "col_sum")
    return out, grad_out


def softmax_rows(x):
    import torch
    _chk_f32(x, "x")
    out = torch.empty_like(x)
    check(lib().agpt_b200_softmax_rows(_dp(x), _dp(out), x.shape[0], x.shape[1], _stream()), "softmax_rows")
    return out


def softmax_backward(s, ds):
    import torch
    _chk_f32(s, "s")
    _chk_f32(ds, "ds")
    out = torch.empty_like(s)
    check(lib().agpt_b200_softmax_bwd(_dp(s), _dp(ds), _dp(out), s.shape[0], s.shape[1], _stream()), "softmax_bwd")
    return out


def embedding_gather(emb, ids32):
    import torch
    _chk_f32(emb, "emb")
    out = torch.empty((ids32.numel(), emb.shape[1]), dtype=torch.float32, device=emb.device)
    check(lib().agpt_b200_embedding_gather(_dp(emb), _dp(ids32), _dp(out), ids32.numel(), emb.shape[1], emb.shape[0], _stream()),
          "embedding_gather")
    return out


def embedding_grad(grad, ids32, vocab, out=None, accumulate=False):
    """Gradient of the embedding table, [vocab, d_model], summed in a fixed order."""
    import torch
    _chk_f32(grad, "grad")
    n, d = grad.shape
    out = torch.zeros((vocab, d), dtype=torch.float32, device=grad.device) if out is None else out
    wsb = check(lib().agpt_b200_embedding_grad_workspace_bytes(n, d, vocab), "embedding_grad_workspace_bytes")
    ws = _workspace(grad.device, "embedding_grad", wsb)
    check(lib().agpt_b200_embedding_grad(_dp(grad), _dp(ids32), _dp(out), n, d, vocab, int(accumulate), _dp(ws), wsb, _stream()),
          "embedding_grad")
    return out


OPTIMIZER_KINDS = {"sgd": 0, "momentum": 1, "rmsprop": 2, "adam": 3}


def optimizer_step(kind, params, grads, m=None, v=None, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, t=1, weight_decay=0.0,
                   clip_norm=0.0, zero_grads=False):
    """Clip, update and decay over flat float32 CUDA buffers, in place.  Returns the gradient norm tensor (one float)
    when clipping is on, else None."""
    import torch
    _chk_f32(params, "params")
    _chk_f32(grads, "grads")
    scratch = None
    if clip_norm > 0:
        scratch = _workspace(params.device, "optimizer", lib().agpt_b200_optimizer_scratch_bytes())
    check(lib().agpt_b200_optimizer_step(OPTIMIZER_KINDS[kind], _dp(params), _dp(grads), _dp(m), _dp(v), params.numel(), lr, beta1,
                                         beta2, eps, t, weight_decay, clip_norm, int(zero_grads), _dp(scratch), _stream()),
          "optimizer_step")
    return scratch.view(torch.float32)[1024:1025] if scratch is not None else None


def suffix_order_gpu(corpus, key_len: int, device: int = 0):
    """(sa, lcp, device milliseconds): start positions 0..n-2 ordered by their first key_len tokens, on the GPU."""
    c = _np_i32(corpus)
    sa, lcp = np.empty(c.size - 1, np.int32), np.empty(c.size - 1, np.int32)
    ms = C.c_float(0)
    check(lib().agpt_b200_suffix_order_gpu(_vp(c), c.size, key_len, device, _vp(sa), _vp(lcp), C.byref(ms)), "suffix_order_gpu")
    return sa, lcp, float(ms.value)


LR_SCHEDULES = {"constant": 0, "cosine": 1, "warmup-cosine": 2}


def compute_lr(base_lr: float, step: int, total_steps: int, warmup_steps: int, schedule: str = "constant") -> float:
    """Learning rate of optimizer step `step` (steps already taken), float32 like the reference."""
    return float(lib().agpt_b200_compute_lr(base_lr, step, total_steps, warmup_steps, LR_SCHEDULES[schedule]))


def device_status() -> int:
    """The current GPU's status word (0 = every kernel ran to completion); synchronises."""
    out = C.c_int32(0)
    check(lib().agpt_b200_device_status(C.byref(out)), "device_status")
    return int(out.value)


def set_gemm_impl(impl: int) -> None:
    """0: mma.sync with three TF32 products; 1 (default): tcgen05 on bfloat16 splits."""
    check(lib().agpt_b200_set_gemm_impl(impl), "set_gemm_impl")


def set_attn_impl(impl: int) -> None:
    """1 = tensor-core kernels (default), 0 = FP32 FMA kernels."""
    check(lib().agpt_b200_set_attn_impl(impl), "set_attn_impl")


def set_attn_variant(whole_tile: bool = True, bwd_warps: int = 4) -> None:
    """Tensor-core kernels for a float32 store and head_dim 32: the whole-tile pair (default) or the chunked pair;
    warps per block of the whole-tile backward (4, 6 or 8)."""
    check(lib().agpt_b200_set_attn_variant(int(bool(whole_tile)), bwd_warps), "set_attn_variant")


def static_scratch_bytes() -> int:
    return int(lib().agpt_b200_static_scratch_bytes())


def attn_backward_static(plan: WalkerPlan, q, k, v, out, lse, dout, n_heads: int, dq, dk, dv, scale: float | None = None):
    """attn_backward for callers that cannot allocate: the partial dK/dV rows go to the library's built-in
    64 MiB device array, so no workspace is passed and the call allocates nothing (the three gradient
    tensors are the caller's).  Plans needing more scratch than the array holds raise AgptError."""
    _chk_f32(q, "q")
    _chk_f32(dout, "dout")
    n, D = q.shape
    hd = D // n_heads
    scale = 1.0 / math.sqrt(hd) if scale is None else scale
    need = plan.workspace_bytes(D)
    if need > static_scratch_bytes():           # the entry point's own first check; made here too so that it precedes the shape checks
        raise AgptError(f"attn_bwd_static: the plan needs {need} bytes of scratch, the built-in array holds {static_scratch_bytes()}")
    validate_attn_args(plan, n_heads, [("q", q), ("out", out), ("dout", dout), ("dq", dq), ("dk", dk), ("dv", dv)],
                       [("k", k), ("v", v)], lse)
    check(lib().agpt_b200_attn_bwd_static(plan._h, _dp(q), _dp(k), _dp(v), _kv_dtype(k), _dp(out), _dp(lse), _dp(dout),
                                          _dp(dq), _dp(dk), _dp(dv), n_heads, hd, scale, _stream()), "attn_bwd_static")
    return dq, dk, dv


def attn_fwd_bwd_host(plan: WalkerPlan, q, k, v, dout, n_heads: int, kv_dtype: int = KV_F32, scale=None,
                      outs=None):
    """Host-buffer step: numpy float32 arrays in and out."""
    n, D = q.shape
    hd = D // n_heads
    scale = 1.0 / math.sqrt(hd) if scale is None else scale
    if outs is None:
        outs = [np.empty((n, D), np.float32), np.empty((n, n_heads), np.float32)] + \
               [np.empty((n, D), np.float32) for _ in range(3)]
    o, lse, dq, dk, dv = outs
    check(lib().agpt_b200_attn_fwd_bwd_host(plan._h, _vp(q), _vp(k), _vp(v), _vp(dout), _vp(o), _vp(lse), _vp(dq),
                                            _vp(dk), _vp(dv), kv_dtype, n_heads, hd, scale), "attn_fwd_bwd_host")
    return o, lse, dq, dk, dv


def loss_per_query(logits, query_to_node, query_offsets, radix_ids, token_ids, counts_offset, counts_tok,
                   counts_val, mass_weights=None, entropy_lambda: float = 0.0, intermediate_weight: float = 1.0,
                   ce_only: bool = False):
    import torch
    _chk_f32(logits, "logits")
    T, V = logits.shape
    g = torch.empty_like(logits)
    loss = torch.empty(T, dtype=torch.float32, device=logits.device)
    check(lib().agpt_b200_loss_per_query(_dp(logits), _dp(query_to_node), _dp(query_offsets), _dp(radix_ids),
                                         _dp(token_ids), _dp(counts_offset), _dp(counts_tok), _dp(counts_val),
                                         _dp(mass_weights), _dp(g), _dp(loss), T, V, entropy_lambda,
                                         intermediate_weight, int(ce_only), _stream()), "loss_per_query")
    return loss, g


def loss_per_node(logits, node_ids, counts_offset, counts_tok, counts_val):
    import torch
    _chk_f32(logits, "logits")
    N, V = logits.shape
    g = torch.empty_like(logits)
    loss = torch.empty(N, dtype=torch.float32, device=logits.device)
    check(lib().agpt_b200_loss_per_node(_dp(logits), _dp(node_ids), _dp(counts_offset), _dp(counts_tok),
                                        _dp(counts_val), _dp(g), _dp(loss), N, V, _stream()), "loss_per_node")
    return loss, g


MASS_MODES = {"off": 0, "log": 1, "sqrt": 2, "linear": 3}


def mass_weights_by_unit(edge_mass, edge_len, unit_of_node, counted, n_units: int, mode: str = "linear") -> np.ndarray:
    """Per-query mass weights where the mean is taken inside each unit (a root-child or bigram subtree) instead of over
    whatever rows share a launch: the weights then do not depend on how units are packed or spread over ranks.
    edge_mass, edge_len, unit_of_node, counted: one entry per loss node; nodes with counted == False (context rows)
    get a weight but do not enter the mean.  Computed by the library (agpt_b200_mass_weights)."""
    em, el = _np_i32(edge_mass), _np_i32(edge_len)
    un = None if unit_of_node is None else _np_i32(unit_of_node)
    inc = None if counted is None else np.ascontiguousarray(counted, dtype=np.uint8)
    out = np.empty(int(el.sum()), np.float32)
    check(lib().agpt_b200_mass_weights(_vp(em), _vp(el), None if un is None else _vp(un), None if inc is None else _vp(inc),
                                       em.size, max(int(n_units), 1), MASS_MODES[mode], _vp(out)), "mass_weights")
    return out


def mass_weights(edge_mass, edge_len, mode: str = "linear") -> np.ndarray:
    """Per-query mass weights of one chunk: f(edge_mass) / mean over the chunk's queries
    (float32 arithmetic with a float64 running total, like the reference's host loop)."""
    return mass_weights_by_unit(edge_mass, edge_len, None, None, 1, mode)


# legacy kernel boundary -------------------------------------------------------------------
def legacy_attention(q, k, v, kv_offsets, kv_lengths, n_heads, head_dim, max_len, scale, query_to_node=None,
                     query_offsets=None):
    import torch
    T = q.numel() // (n_heads * head_dim)
    out = torch.empty(T * n_heads * head_dim, dtype=torch.float32, device=q.device)
    w = torch.empty(T * n_heads * max_len, dtype=torch.float32, device=q.device)
    if query_to_node is None:
        lib().cuda_batched_varlen_attention(_dp(q), _dp(k), _dp(v), _dp(kv_offsets), _dp(kv_lengths), _dp(out), _dp(w),
                                            T, n_heads, head_dim, max_len, scale)
    else:
        lib().cuda_batched_varlen_attention_L_queries(_dp(q), _dp(k), _dp(v), _dp(query_to_node), _dp(query_offsets),
                                                      _dp(kv_offsets), _dp(kv_lengths), _dp(out), _dp(w), T, n_heads,
                                                      head_dim, max_len, scale)
    lib().cuda_sync()
    return out, w


def legacy_attention_backward(q, k, v, w, d_out, kv_offsets, kv_lengths, n_heads, head_dim, max_len, scale,
                              query_to_node=None, query_offsets=None):
    import torch
    T = q.numel() // (n_heads * head_dim)
    dq = torch.empty_like(q)
    if query_to_node is None:
        dk = torch.empty_like(k)
        dv = torch.empty_like(v)
        lib().cuda_batched_varlen_attention_backward(_dp(q), _dp(k), _dp(v), _dp(w), _dp(d_out), _dp(kv_offsets),
                                                     _dp(kv_lengths), _dp(dq), _dp(dk), _dp(dv), T, n_heads, head_dim,
                                                     max_len, scale)
    else:
        dk = torch.zeros_like(k)
        dv = torch.zeros_like(v)
        lib().cuda_batched_varlen_attention_L_queries_backward(_dp(q), _dp(k), _dp(v), _dp(w), _dp(d_out),
                                                               _dp(query_to_node), _dp(query_offsets), _dp(kv_offsets),
                                                               _dp(kv_lengths), _dp(dq), _dp(dk), _dp(dv), T, n_heads,
                                                               head_dim, max_len, scale)
    lib().cuda_sync()
    return dq, dk, dv
