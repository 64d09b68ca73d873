"""ctypes front end of the CPU oracle (``oracle/agpt_oracle.c``).

Test infrastructure only: the parity tests, the smoke check and the CPU-baseline leg of
the benchmark import this module; nothing in the ``agpt_b200`` package does.  Every
function is a thin wrapper around the C restatement, which cites the reference
file:line each routine follows.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libagpt_oracle.so")


def build(force: bool = False) -> str:
    """Compile the C restatement into ``oracle/libagpt_oracle.so``."""
    src = os.path.join(_HERE, "agpt_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(
            ["gcc", "-O3", "-march=native", "-fopenmp", "-fPIC", "-shared", "-fvisibility=hidden",
             "-o", _SO, src, "-lm"])
    return _SO


class _Leveled(C.Structure):
    _fields_ = [("n_nodes", C.c_int32), ("n_levels", C.c_int32),
                ("parent", C.POINTER(C.c_int32)), ("token", C.POINTER(C.c_int32)),
                ("depth", C.POINTER(C.c_int32)), ("level_start", C.POINTER(C.c_int32)),
                ("cnt_off", C.POINTER(C.c_int64)), ("cnt_tok", C.POINTER(C.c_int32)),
                ("cnt_val", C.POINTER(C.c_int32)), ("first_child", C.POINTER(C.c_int32)),
                ("child_count", C.POINTER(C.c_int32))]


class _Radix(C.Structure):
    _fields_ = [("radix_count", C.c_int32), ("n_depth_files", C.c_int32),
                ("total_edge_chars", C.c_int64),
                ("parent", C.POINTER(C.c_int32)), ("first_char_depth", C.POINTER(C.c_int32)),
                ("edge_len", C.POINTER(C.c_int32)), ("edge_mass", C.POINTER(C.c_int32)),
                ("endpoint_depth", C.POINTER(C.c_int32)), ("subtree_key", C.POINTER(C.c_int32)),
                ("endpoint_leveled_id", C.POINTER(C.c_int32)),
                ("edge_off", C.POINTER(C.c_int64)), ("edge_tok", C.POINTER(C.c_int32)),
                ("cnt_off", C.POINTER(C.c_int64)), ("cnt_tok", C.POINTER(C.c_int32)),
                ("cnt_val", C.POINTER(C.c_int32)),
                ("edge_start", C.POINTER(C.c_int32)), ("anc_off", C.POINTER(C.c_int64)),
                ("anc_ids", C.POINTER(C.c_int32))]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        L.orc_token_hash.restype = C.c_uint64
        L.orc_leveled_build.restype = C.POINTER(_Leveled)
        L.orc_radix_build.restype = C.POINTER(_Radix)
        L.orc_num_threads.restype = C.c_int
        _lib = L
    return _lib


def _p(a, t=None):
    if a is None:
        return None
    return a.ctypes.data_as(C.c_void_p)


def _arr(ptr, n, dtype):
    if n == 0:
        return np.zeros(0, dtype=dtype)
    return np.ctypeslib.as_array(ptr, shape=(n,)).astype(dtype, copy=True)


def i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def token_hash(tokens) -> int:
    t = i32(tokens)
    return int(lib().orc_token_hash(_p(t), C.c_int64(t.size)))


class Leveled:
    """Leveled trie arrays as ``streaming_leveled_builder.cr`` would number them."""

    def __init__(self, corpus, max_depth: int):
        c = i32(corpus)
        h = lib().orc_leveled_build(_p(c), C.c_int32(c.size), C.c_int32(max_depth))
        s = h.contents
        n = s.n_nodes
        self.n_nodes, self.n_levels = n, s.n_levels
        self.parent = _arr(s.parent, n, np.int32)
        self.token = _arr(s.token, n, np.int32)
        self.depth = _arr(s.depth, n, np.int32)
        self.level_start = _arr(s.level_start, s.n_levels + 1, np.int32)
        self.cnt_off = _arr(s.cnt_off, n + 1, np.int64)
        nc = int(self.cnt_off[-1])
        self.cnt_tok = _arr(s.cnt_tok, nc, np.int32)
        self.cnt_val = _arr(s.cnt_val, nc, np.int32)
        self._h = h

    def close(self):
        if self._h is not None:
            lib().orc_leveled_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Radix:
    """Radix trie as ``streaming_radix_builder.cr`` emits it, plus the trainer's char index."""

    def __init__(self, leveled: Leveled, subtree_level=1, prune_min_mass=1, prune_min_depth=4):
        h = lib().orc_radix_build(leveled._h, C.c_int32(subtree_level), C.c_int32(prune_min_mass),
                                  C.c_int32(prune_min_depth))
        s = h.contents
        R = s.radix_count
        self.radix_count, self.n_depth_files = R, s.n_depth_files
        self.total_edge_chars = int(s.total_edge_chars)
        for name in ("parent", "first_char_depth", "edge_len", "edge_mass", "endpoint_depth",
                     "subtree_key", "endpoint_leveled_id", "edge_start"):
            setattr(self, name, _arr(getattr(s, name), R, np.int32))
        self.edge_off = _arr(s.edge_off, R + 1, np.int64)
        self.edge_tok = _arr(s.edge_tok, self.total_edge_chars, np.int32)
        self.cnt_off = _arr(s.cnt_off, R + 1, np.int64)
        nc = int(self.cnt_off[-1])
        self.cnt_tok = _arr(s.cnt_tok, nc, np.int32)
        self.cnt_val = _arr(s.cnt_val, nc, np.int32)
        self.anc_off = _arr(s.anc_off, R + 1, np.int64)
        self.anc_ids = _arr(s.anc_ids, int(self.anc_off[-1]), np.int32)
        self._h = h

    def write_dir(self, path, corpus_tokens, vocab, corpus_hash, tag="char.sorted_unique.v1"):
        os.makedirs(path, exist_ok=True)
        rc = lib().orc_radix_write_dir(self._h, path.encode(), C.c_int32(corpus_tokens), C.c_int32(vocab),
                                       C.c_uint64(corpus_hash), tag.encode())
        if rc != 0:
            raise OSError("orc_radix_write_dir failed")

    def write_subtree_files(self, path):
        """subtrees/radix_subtree_KKKKKK.bin and manifest.bin as the reference's builder streams them
        (src/agpt/streaming_radix_builder.cr:257-276 header and records in emission order, :315-330 header patch and
        manifest order, :396-408 record, :413-426 manifest): header u32 magic, i32 version 2, i32 key, i32 records,
        i64 edge chars, i32 deepest endpoint; records with GLOBAL radix ids."""
        import struct
        os.makedirs(os.path.join(path, "subtrees"), exist_ok=True)
        magic = 0x52445841
        keys = {}
        for r in range(1, self.radix_count):
            keys.setdefault(int(self.subtree_key[r]), []).append(r)
        manifest = []
        for key, ids in keys.items():
            body = bytearray()
            chars, max_ep = 0, 0
            for r in ids:
                el = int(self.edge_len[r])
                body += struct.pack("<4i", r, int(self.parent[r]), int(self.first_char_depth[r]), el)
                body += np.asarray(self.edge_tok[self.edge_off[r]:self.edge_off[r] + el], "<i4").tobytes()
                c0, c1 = int(self.cnt_off[r]), int(self.cnt_off[r + 1])
                body += struct.pack("<2i", int(self.edge_mass[r]), c1 - c0)
                for e in range(c0, c1):
                    body += struct.pack("<2i", int(self.cnt_tok[e]), int(self.cnt_val[e]))
                chars += el
                max_ep = max(max_ep, int(self.endpoint_depth[r]))
            with open(os.path.join(path, "subtrees", "radix_subtree_%06d.bin" % key), "wb") as f:
                f.write(struct.pack("<I3iqi", magic, 2, key, len(ids), chars, max_ep))
                f.write(bytes(body))
            manifest.append((key, len(ids), chars, max_ep))
        manifest.sort()
        with open(os.path.join(path, "manifest.bin"), "wb") as f:
            f.write(struct.pack("<I2i", magic, 2, len(manifest)))
            for key, cnt, chars, max_ep in manifest:
                f.write(struct.pack("<2iqi", key, cnt, chars, max_ep))

    def char_tree(self):
        """Char-position tree: parent char position of every edge char (-1 under the root),
        in the trainer's char numbering (``agpt_train.cu:832``); plus token and depth."""
        n = self.total_edge_chars
        par = np.full(n, -1, np.int32)
        tok = np.zeros(n, np.int32)
        dep = np.zeros(n, np.int32)
        for r in range(1, self.radix_count):
            s, L = int(self.edge_start[r]), int(self.edge_len[r])
            p = int(self.parent[r])
            par[s] = -1 if p == 0 else int(self.edge_start[p] + self.edge_len[p] - 1)
            if L > 1:
                par[s + 1:s + L] = np.arange(s, s + L - 1, dtype=np.int32)
            tok[s:s + L] = self.edge_tok[self.edge_off[r]:self.edge_off[r + 1]]
            dep[s:s + L] = self.first_char_depth[r] + np.arange(L, dtype=np.int32)
        return par, tok, dep

    def close(self):
        if self._h is not None:
            lib().orc_radix_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def rope_table(max_seq, dim, base=10000.0):
    c = np.zeros((max_seq, dim), np.float32)
    s = np.zeros((max_seq, dim), np.float32)
    lib().orc_rope_table(_p(c), _p(s), C.c_int(max_seq), C.c_int(dim), C.c_float(base))
    return c, s


def rope_apply(x, pos, cos, sin, inverse=False):
    """x: [rows, dim] float32 (modified copy returned); pos: [rows]."""
    x = f32(x).copy()
    pos = i32(pos)
    lib().orc_rope_apply(_p(x), _p(pos), _p(f32(cos)), _p(f32(sin)), C.c_int64(x.shape[0]),
                         C.c_int(x.shape[1]), C.c_int(1 if inverse else 0))
    return x


def tree_depth(parent):
    parent = i32(parent)
    d = np.zeros(parent.size, np.int32)
    for i in range(parent.size):
        d[i] = 1 if parent[i] < 0 else d[parent[i]] + 1
    return d


def tree_depth_fast(parent):
    """Depths for parent[i] < i trees without a Python loop over nodes (level sweeps)."""
    parent = i32(parent)
    d = np.where(parent < 0, 1, 0).astype(np.int32)
    todo = d == 0
    while todo.any():
        idx = np.nonzero(todo)[0]
        pd = d[parent[idx]]
        ok = pd > 0
        d[idx[ok]] = pd[ok] + 1
        todo[idx[ok]] = False
    return d


def weight_offsets(depth, H):
    off = np.zeros(depth.size + 1, np.int64)
    np.cumsum(depth.astype(np.int64) * H, out=off[1:])
    return off


def attn_fwd(parent, H, hd, q, k, v, grouped=False, save_weights=True):
    parent = i32(parent)
    n = parent.size
    q, k, v = f32(q), f32(k), f32(v)
    depth = tree_depth_fast(parent)
    md = int(depth.max()) if n else 1
    w_off = weight_offsets(depth, H)
    out = np.zeros((n, H * hd), np.float32)
    w = np.zeros(int(w_off[-1]), np.float32) if save_weights else None
    if grouped:
        order = np.argsort(parent, kind="stable").astype(np.int32)
        ps = parent[order]
        starts = np.concatenate([[0], np.nonzero(np.diff(ps))[0] + 1, [n]]).astype(np.int32) if n else np.zeros(1, np.int32)
        # children of the key-less root (parent -1) form a single group with an empty prefix
        rc = lib().orc_attn_fwd_grouped(C.c_int32(n), _p(parent), C.c_int32(starts.size - 1), _p(starts),
                                        _p(order), C.c_int(H), C.c_int(hd), _p(q), _p(k), _p(v), _p(out),
                                        _p(w), _p(w_off), C.c_int(md))
    else:
        rc = lib().orc_attn_fwd_per_node(C.c_int32(n), _p(parent), C.c_int(H), C.c_int(hd), _p(q), _p(k),
                                         _p(v), _p(out), _p(w), _p(w_off), C.c_int(md))
    if rc != 0:
        raise RuntimeError("oracle attention forward failed (bad parent chain)")
    return out, w, w_off, depth


def attn_bwd(parent, H, hd, q, k, v, w, w_off, d_out, accumulate_ancestors=True, unit_off=None, edge_id=None):
    """accumulate_ancestors: True / 1 = every ancestor row receives its dK/dV (persistent accumulators), False / 0 =
    none does (local depth), 2 = only the ancestors on the node's own radix edge (edge_id[a] == edge_id[i])."""
    parent = i32(parent)
    n = parent.size
    q, k, v, d_out = f32(q), f32(k), f32(v), f32(d_out)
    depth = tree_depth_fast(parent)
    md = int(depth.max()) if n else 1
    dq = np.zeros((n, H * hd), np.float32)
    dk = np.zeros_like(dq)
    dv = np.zeros_like(dq)
    uo = i32(unit_off) if unit_off is not None else None
    rc = lib().orc_attn_bwd(C.c_int32(n), _p(parent), C.c_int(H), C.c_int(hd), _p(q), _p(k), _p(v),
                            _p(f32(w)), _p(np.ascontiguousarray(w_off, np.int64)), _p(d_out), _p(dq), _p(dk),
                            _p(dv), C.c_int(md), C.c_int(int(accumulate_ancestors)),
                            C.c_int32(0 if uo is None else uo.size - 1), _p(uo),
                            _p(i32(edge_id)) if edge_id is not None else None)
    if rc != 0:
        raise RuntimeError("oracle attention backward failed")
    return dq, dk, dv


def bwd_head_matrix(K, V, w, qv, go, accum_dk, accum_dv):
    K, V = f32(K), f32(V)
    ln, hd = K.shape
    dq = np.zeros(hd, np.float32)
    dkf = np.zeros((ln, hd), np.float32)
    dvf = np.zeros((ln, hd), np.float32)
    lib().orc_attn_bwd_head_matrix(C.c_int(ln), C.c_int(hd), _p(K), _p(V), _p(f32(w)), _p(f32(qv)), _p(f32(go)),
                                   _p(f32(accum_dk)), _p(f32(accum_dv)), _p(dq), _p(dkf), _p(dvf))
    return dq, dkf, dvf


def bwd_head_optimized(K, V, w, qv, go, accum_dk, accum_dv, anc_dk, anc_dv):
    K, V = f32(K), f32(V)
    ln, hd = K.shape
    dq = np.zeros(hd, np.float32)
    dkc = np.zeros(hd, np.float32)
    dvc = np.zeros(hd, np.float32)
    anc_dk = f32(anc_dk).copy()
    anc_dv = f32(anc_dv).copy()
    lib().orc_attn_bwd_head_optimized(C.c_int(ln), C.c_int(hd), _p(K), _p(V), _p(f32(w)), _p(f32(qv)),
                                      _p(f32(go)), _p(f32(accum_dk)), _p(f32(accum_dv)), _p(dq), _p(dkc),
                                      _p(dvc), _p(anc_dk), _p(anc_dv))
    return dq, dkc, dvc, anc_dk, anc_dv


def packed_attn_fwd(q, k, v, kv_offsets, kv_lengths, H, hd, max_len, scale, query_to_node=None,
                    query_offsets=None):
    q, k, v = f32(q), f32(k), f32(v)
    T = q.size // (H * hd)
    out = np.zeros(T * H * hd, np.float32)
    w = np.zeros(T * H * max_len, np.float32)
    lib().orc_packed_attn_fwd(_p(q), _p(k), _p(v), _p(i32(query_to_node)) if query_to_node is not None else None,
                              _p(i32(query_offsets)) if query_offsets is not None else None,
                              _p(i32(kv_offsets)), _p(i32(kv_lengths)), _p(out), _p(w), C.c_int(T), C.c_int(H),
                              C.c_int(hd), C.c_int(max_len), C.c_float(scale))
    return out, w


def packed_attn_bwd(q, k, v, w, d_out, kv_offsets, kv_lengths, H, hd, max_len, scale, query_to_node=None,
                    query_offsets=None):
    q, k, v, w, d_out = f32(q), f32(k), f32(v), f32(w), f32(d_out)
    T = q.size // (H * hd)
    dq = np.zeros(T * H * hd, np.float32)
    dk = np.zeros(k.size, np.float32)
    dv = np.zeros(v.size, np.float32)
    lib().orc_packed_attn_bwd(_p(q), _p(k), _p(v), _p(w), _p(d_out),
                              _p(i32(query_to_node)) if query_to_node is not None else None,
                              _p(i32(query_offsets)) if query_offsets is not None else None,
                              _p(i32(kv_offsets)), _p(i32(kv_lengths)), _p(dq), _p(dk), _p(dv), C.c_int(T),
                              C.c_int(H), C.c_int(hd), C.c_int(max_len), C.c_float(scale))
    return dq, dk, dv


def loss_per_query(logits, query_to_node, query_offsets, radix_ids, token_ids, counts_offset, counts_tok,
                   counts_val, mass_weights=None, entropy_lambda=0.0, intermediate_weight=1.0, ce_only=False):
    logits = f32(logits)
    T, V = logits.shape
    g = np.zeros((T, V), np.float32)
    loss = np.zeros(T, np.float32)
    mw = f32(mass_weights) if mass_weights is not None else None
    lib().orc_loss_per_query(_p(logits), _p(i32(query_to_node)), _p(i32(query_offsets)), _p(i32(radix_ids)),
                             _p(i32(token_ids)), _p(i32(counts_offset)), _p(i32(counts_tok)), _p(i32(counts_val)),
                             _p(mw), _p(g), _p(loss), C.c_int(T), C.c_int(V), C.c_float(entropy_lambda),
                             C.c_float(intermediate_weight), C.c_int(1 if ce_only else 0))
    return loss, g


def loss_per_node(logits, node_ids, counts_offset, counts_tok, counts_val):
    logits = f32(logits)
    N, V = logits.shape
    g = np.zeros((N, V), np.float32)
    loss = np.zeros(N, np.float32)
    lib().orc_loss_per_node(_p(logits), _p(i32(node_ids)), _p(i32(counts_offset)), _p(i32(counts_tok)),
                            _p(i32(counts_val)), _p(g), _p(loss), C.c_int(N), C.c_int(V))
    return loss, g


def loss_crystal(logits, counts_offset, counts_tok, counts_val, lam=0.0):
    logits = f32(logits)
    N, V = logits.shape
    g = np.zeros((N, V), np.float32)
    loss = np.zeros(N, np.float64)
    lib().orc_loss_crystal(_p(logits), _p(i32(counts_offset)), _p(i32(counts_tok)), _p(i32(counts_val)), _p(g),
                           _p(loss), C.c_int(N), C.c_int(V), C.c_double(lam))
    return loss, g


def mass_weights(edge_mass, edge_len, mode):
    """mode: 0 off, 1 log1p, 2 sqrt, 3 linear."""
    em, el = i32(edge_mass), i32(edge_len)
    out = np.zeros(int(el.sum()), np.float32)
    lib().orc_mass_weights(_p(em), _p(el), C.c_int(em.size), C.c_int(mode), _p(out))
    return out


def layer_norm_fwd(x, gamma, beta):
    x = f32(x)
    rows, cols = x.shape
    y, norm, sinv = np.zeros_like(x), np.zeros_like(x), np.zeros(rows, np.float32)
    lib().orc_layer_norm_fwd(_p(x), _p(y), _p(norm), _p(sinv), _p(f32(gamma)), _p(f32(beta)), C.c_int64(rows), C.c_int(cols))
    return y, norm, sinv


def layer_norm_bwd(grad, norm, sinv, gamma):
    grad = f32(grad)
    rows, cols = grad.shape
    dx, dg, db = np.zeros_like(grad), np.zeros(cols, np.float32), np.zeros(cols, np.float32)
    lib().orc_layer_norm_bwd(_p(grad), _p(f32(norm)), _p(f32(sinv)), _p(f32(gamma)), _p(dx), _p(dg), _p(db), C.c_int64(rows),
                             C.c_int(cols))
    return dx, dg, db


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(C.c_int(n))


def num_threads() -> int:
    return int(lib().orc_num_threads())


# ---- dense-step row kernels and optimizer rules (numpy restatements; float32 arithmetic) ------------------------------
# Follow the reference's CPU statements of the same steps: bias add and ReLU of the feed-forward block
# (src/agpt/incremental_forward.cr:165-217), the bias gradient as a column sum (src/cuda/agpt_train.cu:1771-1790),
# softmax backward s*(ds - sum s*ds) (src/agpt/batched_depth_backward.cr:605-695 uses the same identity per head),
# and the optimizer call order clip -> update -> decay (src/cuda/agpt_train.cu:5135-5162).

def bias_relu(x, bias, relu):
    y = (f32(x) + f32(bias)[None, :]).astype(np.float32)
    if not relu:
        return y, None
    return np.maximum(y, np.float32(0)), (y > 0).astype(np.float32)


def relu_bwd(grad, mask):
    return np.where(f32(mask) > 0, f32(grad), np.float32(0)).astype(np.float32)


def col_sum(grad):
    return f32(grad).astype(np.float64).sum(axis=0)


def softmax_rows(x):
    x = f32(x).astype(np.float64)
    e = np.exp(x - x.max(axis=1, keepdims=True))
    return e / e.sum(axis=1, keepdims=True)


def softmax_bwd(s, ds):
    s, ds = f32(s).astype(np.float64), f32(ds).astype(np.float64)
    return s * (ds - (s * ds).sum(axis=1, keepdims=True))


def embedding_grad(grad, ids, vocab):
    out = np.zeros((vocab, grad.shape[1]), np.float64)
    np.add.at(out, np.asarray(ids)[np.asarray(ids) >= 0], f32(grad).astype(np.float64)[np.asarray(ids) >= 0])
    return out


def optimizer_step(kind, p, g, m, v, lr, beta1, beta2, eps, t, weight_decay=0.0, clip_norm=0.0):
    """One step in float32, element by element as the kernels do.  Returns (p, m, v, gradient norm)."""
    one = np.float32(1)
    p, g = f32(p).copy(), f32(g).copy()
    m = None if m is None else f32(m).copy()
    v = None if v is None else f32(v).copy()
    lr, beta1, beta2, eps = np.float32(lr), np.float32(beta1), np.float32(beta2), np.float32(eps)
    norm = float(np.sqrt((g.astype(np.float64) ** 2).sum()))
    if clip_norm > 0 and norm > clip_norm:
        g = (g * np.float32(clip_norm / norm)).astype(np.float32)
    if kind == "sgd":
        p = p - lr * g
    elif kind == "momentum":
        m = beta1 * m + g
        p = p - lr * m
    elif kind == "rmsprop":
        v = beta2 * v + (one - beta2) * g * g
        p = p - lr * g / (np.sqrt(v) + eps)
    elif kind == "adam":
        m = beta1 * m + (one - beta1) * g
        v = beta2 * v + (one - beta2) * g * g
        bc1 = one - np.float32(np.float32(beta1) ** np.float32(t))
        bc2 = one - np.float32(np.float32(beta2) ** np.float32(t))
        p = p - lr * (m / bc1) / (np.sqrt(v / bc2) + eps)
    else:
        raise ValueError(kind)
    p = p.astype(np.float32)
    if weight_decay > 0:
        p = (p - lr * np.float32(weight_decay) * p).astype(np.float32)
    return p, m, v, norm


# ---- stochastic training units ("lightning" sampling) ------------------------------------------------------------------
# Restates src/cuda/agpt_train.cu:188-200 (generator), :3928-3943 (child adjacency in id order) and :4060-4241 (the four
# samplers, the node set of a sample, its endpoint-depth bucket order).  Plain Python: for small tries only.

def xorshift32(state):
    x = state & 0xFFFFFFFF
    x ^= (x << 13) & 0xFFFFFFFF
    x ^= x >> 17
    x ^= (x << 5) & 0xFFFFFFFF
    return x if x else 1


def lightning_sample(parent, edge_mass, first_char_depth, edge_len, sampler, steps, state, p_stop=0.3, max_mass=0):
    """Returns ([(sampled id, ancestor count, summed mass, node ids)], new generator state)."""
    R = len(parent)
    kids = [[] for _ in range(R)]
    for r in range(1, R):
        kids[int(parent[r])].append(r)

    def unit():
        nonlocal state
        state = xorshift32(state)
        return float(np.float32(state) / np.float32(4294967296.0))

    def below(n):
        nonlocal state
        state = xorshift32(state)
        return state % n

    def root_child():
        return kids[0][below(len(kids[0]))] if kids[0] else 0

    out = []
    for _ in range(steps):
        pick = 0
        if sampler in (3, 4):
            stop = np.float32(0.0 if sampler == 4 else p_stop)
            cur = 0
            while True:
                forced = max_mass > 0 and cur != 0 and int(edge_mass[cur]) > max_mass
                if cur != 0 and stop > 0 and not forced and np.float32(unit()) < stop:
                    break
                ch = kids[cur]
                if not ch:
                    break
                tot = float(sum(float(edge_mass[c]) for c in ch))
                if tot <= 0.0:
                    nxt = ch[below(len(ch))]
                else:
                    u = unit() * tot
                    acc, nxt = 0.0, ch[-1]
                    for c in ch:
                        acc += float(edge_mass[c])
                        if u <= acc:
                            nxt = c
                            break
                cur = nxt
            pick = cur
        elif sampler == 1:
            if R > 1:
                pick = 1 + below(R - 1)
        else:
            pick = root_child()
        if pick == 0:
            pick = root_child()
        anc, c = [], int(parent[pick])
        while c > 0:
            anc.append(c)
            c = int(parent[c])
        anc.reverse()
        if sampler == 4:
            nodes, n_anc = anc + [pick], 0
        else:
            nodes, n_anc = anc + [pick], len(anc)
            head = len(anc)
            while head < len(nodes):
                nodes.extend(kids[nodes[head]])
                head += 1
        mass = float(sum(float(edge_mass[x]) for x in nodes))
        ep = lambda x: int(first_char_depth[x]) + int(edge_len[x]) - 1  # noqa: E731
        nodes = sorted(nodes, key=ep)              # sorted() is stable, like the reference's bucket pass
        out.append((pick, n_anc, mass, nodes))
    return out, state


def compute_lr(base_lr, step, total_steps, warmup_steps, schedule):
    """src/cuda/agpt_train.cu:202-216 in float32; schedule 0 constant, 1 cosine, 2 warm-up then cosine."""
    f = np.float32
    if total_steps <= 1 or schedule == 0:
        return f(base_lr)
    if schedule == 2 and step < warmup_steps:
        return f(f(base_lr) * (f(step + 1) / f(warmup_steps)))
    cos_start = warmup_steps if schedule == 2 else 0
    if total_steps <= cos_start:
        return f(base_lr)
    progress = min(f(step - cos_start) / f(total_steps - cos_start), f(1.0))
    return f(f(0.5) * f(base_lr) * (f(1.0) + np.cos(f(f(3.14159265358979323846) * progress), dtype=np.float32)))


def lightning_lr_weights(masses, mode):
    """src/cuda/agpt_train.cu:4276-4300 as a plain loop; mode 0 off, 1 log, 2 sqrt, 3 linear."""
    import math
    comp = []
    for m in masses:
        m = float(m)
        comp.append(math.log(1.0 + m) if mode == 1 else ((math.sqrt(m) if m > 0.0 else 0.0) if mode == 2 else (m if mode == 3 else 1.0)))
    total = 0.0
    for c in comp:
        total += c
    mean = total / len(comp) if (comp and total > 0.0) else 1.0
    return [c / mean for c in comp]
