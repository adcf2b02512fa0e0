"""The committed C0 vectors (tests/golden/c0_tiny.npz) against the CPU oracle: integer results and
logits must be reproduced exactly, so that any change of the oracle's arithmetic is visible."""
import importlib.util
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def load_generator():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_oracle_reproduces_the_committed_vectors():
    gold = np.load(os.path.join(HERE, "golden", "c0_tiny.npz"))
    now = load_generator().build()
    assert sorted(gold.files) == sorted(now.keys())
    for key in gold.files:
        want, got = gold[key], np.asarray(now[key])
        assert want.shape == got.shape, key
        if want.dtype.kind in "iu":
            assert np.array_equal(want, got), key
        else:
            # same source and compiler flags give the same bits; allow the last ulps for a different libm
            assert np.allclose(want, got, rtol=1e-6, atol=1e-6), key
    assert int(gold["chain_accepted"][0]) == 2 and int(gold["tree_accepted"][0]) == 3
    assert gold["tree_path"].tolist() == [2, 8, 12]
    assert gold["lookup_draft"].tolist() == [8, 5, 6, 7]
