"""MGPT checkpoint format: round trip, and the reference's own data/input.model when it is mounted."""
import filecmp
import os

import numpy as np
import pytest

from agpt_b200 import model_file as MF
from tests.conftest import REFERENCE_ROOT

REF_MODEL = os.path.join(REFERENCE_ROOT, "data", "input.model")


def test_round_trip(tmp_path):
    m = MF.random_init(32, 2, 3, 17, 64, seed=5)
    p = str(tmp_path / "m.model")
    MF.save(p, m)
    assert os.path.getsize(p) == 28 + sum(8 + 4 * r * c for r, c in m.expected_shapes())
    back = MF.load(p)
    assert (back.d_model, back.n_heads, back.n_layers, back.d_ff, back.vocab, back.seq_len) == (32, 2, 3, 128, 17, 64)
    assert len(back.mats) == 1 + 16 * 3 + 4
    for (n1, a), (n2, b) in zip(m.mats, back.mats):
        assert n1 == n2 and np.array_equal(a, b)
    open(p, "r+b").write(b"XXXX")
    with pytest.raises(ValueError):
        MF.load(p)


@pytest.mark.skipif(not os.path.exists(REF_MODEL), reason="reference model file not mounted")
def test_reference_model_file_bytes(tmp_path):
    m = MF.load(REF_MODEL)
    assert (m.d_model, m.n_heads, m.n_layers, m.d_ff, m.vocab, m.seq_len) == (64, 4, 2, 256, 65, 128)
    assert len(m.mats) == 37 and os.path.getsize(REF_MODEL) == 434_248
    out = str(tmp_path / "copy.model")
    MF.save(out, m)
    assert filecmp.cmp(out, REF_MODEL, shallow=False)
