"""MGPT model file: the checkpoint format of the reference trainer, read and written unchanged.

Layout (src/cuda/agpt_train.cu:1209-1296): u32 magic 0x4D475054, i32 d_model, n_heads, n_layers, d_ff,
vocab, seq_len, then 1 + 16*n_layers + 4 matrices, each i32 rows, i32 cols, f32[rows*cols] row-major
([d_in, d_out], y = x W + b), in the order token_emb; per layer wq.w, wq.b, wk.w, wk.b, wv.w, wv.b, wo.w,
wo.b, ln1.gamma, ln1.beta, l1.w, l1.b, l2.w, l2.b, ln2.gamma, ln2.beta; final gamma, beta; out.w, out.b.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

import numpy as np

MAGIC = 0x4D475054
LAYER_NAMES = ("wq.w", "wq.b", "wk.w", "wk.b", "wv.w", "wv.b", "wo.w", "wo.b", "ln1.gamma", "ln1.beta",
               "l1.w", "l1.b", "l2.w", "l2.b", "ln2.gamma", "ln2.beta")


@dataclass
class Model:
    d_model: int
    n_heads: int
    n_layers: int
    d_ff: int
    vocab: int
    seq_len: int
    mats: list = field(default_factory=list)     # [(name, float32 array [rows, cols])] in file order

    def names(self):
        out = ["token_emb"]
        for l in range(self.n_layers):
            out += [f"layer{l}.{n}" for n in LAYER_NAMES]
        return out + ["final.gamma", "final.beta", "out.w", "out.b"]

    def expected_shapes(self):
        D, F, V = self.d_model, self.d_ff, self.vocab
        per = [(D, D), (1, D)] * 4 + [(1, D), (1, D), (D, F), (1, F), (F, D), (1, D), (1, D), (1, D)]
        return [(V, D)] + per * self.n_layers + [(1, D), (1, D), (D, V), (1, V)]

    def get(self, name):
        return dict(self.mats)[name]


def load(path: str) -> Model:
    with open(path, "rb") as f:
        raw = f.read()
    if len(raw) < 28 or struct.unpack_from("<I", raw, 0)[0] != MAGIC:
        raise ValueError(f"{path}: bad model magic")
    d_model, n_heads, n_layers, d_ff, vocab, seq_len = struct.unpack_from("<6i", raw, 4)
    m = Model(d_model, n_heads, n_layers, d_ff, vocab, seq_len)
    off = 28
    for name, shape in zip(m.names(), m.expected_shapes()):
        rows, cols = struct.unpack_from("<2i", raw, off)
        off += 8
        if (rows, cols) != shape:
            raise ValueError(f"{path}: matrix {name} is {rows}x{cols}, expected {shape[0]}x{shape[1]}")
        cnt = rows * cols
        m.mats.append((name, np.frombuffer(raw, dtype="<f4", count=cnt, offset=off).reshape(rows, cols).copy()))
        off += cnt * 4
    if off != len(raw):
        raise ValueError(f"{path}: {len(raw) - off} trailing bytes")
    return m


def save(path: str, m: Model) -> None:
    with open(path, "wb") as f:
        f.write(struct.pack("<I6i", MAGIC, m.d_model, m.n_heads, m.n_layers, m.d_ff, m.vocab, m.seq_len))
        for (name, a), shape in zip(m.mats, m.expected_shapes()):
            a = np.ascontiguousarray(a, dtype="<f4")
            if a.shape != shape:
                raise ValueError(f"matrix {name} has shape {a.shape}, expected {shape}")
            f.write(struct.pack("<2i", *shape))
            f.write(a.tobytes())


def random_init(d_model, n_heads, n_layers, vocab, seq_len, d_ff=None, seed=0, std=0.02) -> Model:
    """Seeded N(0, std) weights, gamma 1, beta and biases 0, in file order."""
    d_ff = 4 * d_model if d_ff is None else d_ff
    m = Model(d_model, n_heads, n_layers, d_ff, vocab, seq_len)
    rng = np.random.default_rng(seed)
    for name, shape in zip(m.names(), m.expected_shapes()):
        if name.endswith("gamma"):
            a = np.ones(shape, np.float32)
        elif name.endswith(".b") or name.endswith("beta"):
            a = np.zeros(shape, np.float32)
        else:
            a = (rng.standard_normal(shape) * std).astype(np.float32)
        m.mats.append((name, a))
    return m
